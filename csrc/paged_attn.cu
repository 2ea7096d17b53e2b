// Paged-KV kernels for the rollout engine (sm_100a).
//   * kv_write: scatter new K/V rows of a step into their cache slots
//   * paged decode attention: one query token per request, GQA, split-KV with a
//     log-sum-exp combine. Decode attention is bound by reading the KV cache once,
//     so the kernel is organised around coalesced 16-byte row reads: per 32-token
//     chunk, lanes first own tokens (q.k scores), then own output dims (p.V).
//
// Cache layout: k_cache / v_cache = [num_slots, Hkv, D] bf16 where slot = page * page_size
// + offset; block_table[b, i] = page id of the i-th page of request b.
#include "common.cuh"

namespace sb {

__global__ void kv_write_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                const int* __restrict__ slots, __nv_bfloat16* __restrict__ k_cache,
                                __nv_bfloat16* __restrict__ v_cache, int T, int row_elems, int k_stride, int v_stride) {
  pdl_wait();  // inputs come from the previous kernel in the stream
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  const uint4* ks = reinterpret_cast<const uint4*>(k + static_cast<size_t>(t) * k_stride);
  const uint4* vs = reinterpret_cast<const uint4*>(v + static_cast<size_t>(t) * v_stride);
  uint4* kd = reinterpret_cast<uint4*>(k_cache + static_cast<size_t>(slot) * row_elems);
  uint4* vd = reinterpret_cast<uint4*>(v_cache + static_cast<size_t>(slot) * row_elems);
  for (int c = threadIdx.x; c < (row_elems >> 3); c += blockDim.x) {
    kd[c] = ks[c];
    vd[c] = vs[c];
  }
}

constexpr int DEC_WARPS = 4;
constexpr int DEC_THREADS = DEC_WARPS * 32;

// grid = (B, Hkv, splits). q: [B, Hq, D] (pitch q_stride per request). G = Hq / Hkv (<= 8).
// Partial results: part_o [B, Hq, splits, D] fp32, part_ml [B, Hq, splits, 2] (max, sum).
template <int D, int G>
__global__ void __launch_bounds__(DEC_THREADS)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                    const int* __restrict__ seq_lens, float* __restrict__ part_o, float* __restrict__ part_ml,
                    int Hq, int Hkv, int page_size, int max_pages, int q_stride, int splits, float scale) {
  constexpr int DPL = D / 32;  // output dims per lane
  __shared__ float q_s[G][D];
  __shared__ float p_s[DEC_WARPS][G][32];
  __shared__ float red_m[DEC_WARPS][G], red_l[DEC_WARPS][G];
  __shared__ float red_o[DEC_WARPS][G][D];

  const int b = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = seq_lens[b];
  const int chunk_tokens = ((len + splits - 1) / splits + 31) & ~31;
  const int t_begin = sp * chunk_tokens;
  const int t_end = min(len, t_begin + chunk_tokens);

  for (int i = threadIdx.x; i < G * D; i += DEC_THREADS) {
    const int g = i / D, d = i % D;
    q_s[g][d] = __bfloat162float(q[static_cast<size_t>(b) * q_stride + static_cast<size_t>(kvh * G + g) * D + d]) * scale;
  }
  __syncthreads();

  float m[G], l[G], acc[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[g][j] = 0.f;
  }
  const int* bt = block_table + static_cast<size_t>(b) * max_pages;
  const size_t row = static_cast<size_t>(Hkv) * D;

  for (int t0 = t_begin + warp * 32; t0 < t_end; t0 += DEC_WARPS * 32) {
    // phase 1: lane = token, scores for the G query heads
    const int tok = t0 + lane;
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = -INFINITY;
    if (tok < t_end) {
      const int slot = bt[tok / page_size] * page_size + tok % page_size;
      const uint4* kr = reinterpret_cast<const uint4*>(k_cache + slot * row + static_cast<size_t>(kvh) * D);
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] = 0.f;
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        const uint4 u = kr[c];
        const float2 a = unpack_bf16x2(u.x), bb = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), dd = unpack_bf16x2(u.w);
        const float kf[8] = {a.x, a.y, bb.x, bb.y, cc.x, cc.y, dd.x, dd.y};
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
          for (int i = 0; i < 8; ++i) s[g] += kf[i] * q_s[g][c * 8 + i];
        }
      }
    }
    // online softmax bookkeeping per head (warp-wide max / sum over the 32 tokens)
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float cm = warp_max(s[g]);
      const float nm = fmaxf(m[g], cm);
      const float p = (tok < t_end) ? __expf(s[g] - nm) : 0.f;
      const float corr = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - nm);
      l[g] = l[g] * corr + warp_sum(p);
#pragma unroll
      for (int j = 0; j < DPL; ++j) acc[g][j] *= corr;
      m[g] = nm;
      p_s[warp][g][lane] = p;
    }
    __syncwarp();
    // phase 2: lane = output dims [lane*DPL, lane*DPL+DPL); walk the chunk's tokens
    const int ntok = min(32, t_end - t0);
    for (int j = 0; j < ntok; ++j) {
      const int tk = t0 + j;
      const int slot = bt[tk / page_size] * page_size + tk % page_size;
      const __nv_bfloat16* vr = v_cache + slot * row + static_cast<size_t>(kvh) * D + lane * DPL;
      float vf[DPL];
      if constexpr (DPL == 2) {
        const float2 t2 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(vr));
        vf[0] = t2.x; vf[1] = t2.y;
      } else if constexpr (DPL == 4) {
        const uint2 u = *reinterpret_cast<const uint2*>(vr);
        const float2 a = unpack_bf16x2(u.x), bb = unpack_bf16x2(u.y);
        vf[0] = a.x; vf[1] = a.y; vf[2] = bb.x; vf[3] = bb.y;
      } else {
#pragma unroll
        for (int i = 0; i < DPL; ++i) vf[i] = __bfloat162float(vr[i]);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float p = p_s[warp][g][j];
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] += p * vf[i];
      }
    }
    __syncwarp();
  }

  // combine the warps of the CTA
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      red_m[warp][g] = m[g];
      red_l[warp][g] = l[g];
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) red_o[warp][g][lane * DPL + i] = acc[g][i];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += DEC_THREADS) {
    const int g = i / D, d = i % D;
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) gm = fmaxf(gm, red_m[w][g]);
    float gl = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float c = (red_m[w][g] == -INFINITY) ? 0.f : __expf(red_m[w][g] - gm);
      gl += red_l[w][g] * c;
      o += red_o[w][g][d] * c;
    }
    const int h = kvh * G + g;
    const size_t base = (static_cast<size_t>(b) * Hq + h) * splits + sp;
    part_o[base * D + d] = o;
    if (d == 0) {
      part_ml[base * 2 + 0] = gm;
      part_ml[base * 2 + 1] = gl;
    }
  }
}

// out[b, h, :] = sum_s part_o * exp(m_s - M) / sum_s l_s exp(m_s - M); also lse (optional).
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      __nv_bfloat16* __restrict__ out, int D, int splits, int out_stride, int Hq) {
  const int bh = blockIdx.x;  // b * Hq + h
  const int b = bh / Hq, h = bh % Hq;
  float gm = -INFINITY;
  for (int s = 0; s < splits; ++s) gm = fmaxf(gm, part_ml[(static_cast<size_t>(bh) * splits + s) * 2]);
  float gl = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(static_cast<size_t>(bh) * splits + s) * 2];
    gl += (ms == -INFINITY) ? 0.f : part_ml[(static_cast<size_t>(bh) * splits + s) * 2 + 1] * __expf(ms - gm);
  }
  const float inv = gl > 0.f ? 1.f / gl : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = part_ml[(static_cast<size_t>(bh) * splits + s) * 2];
      if (ms != -INFINITY) o += part_o[(static_cast<size_t>(bh) * splits + s) * D + d] * __expf(ms - gm);
    }
    out[static_cast<size_t>(b) * out_stride + static_cast<size_t>(h) * D + d] = __float2bfloat16(o * inv);
  }
}

template <int D>
static int launch_decode(int G, dim3 grid, cudaStream_t s, const __nv_bfloat16* q, const __nv_bfloat16* kc,
                         const __nv_bfloat16* vc, const int* bt, const int* sl, float* po, float* pml, int Hq, int Hkv,
                         int page_size, int max_pages, int q_stride, int splits, float scale) {
#define SB_G(GV)                                                                                                  \
  case GV:                                                                                                        \
    paged_decode_kernel<D, GV><<<grid, DEC_THREADS, 0, s>>>(q, kc, vc, bt, sl, po, pml, Hq, Hkv, page_size, max_pages, \
                                                            q_stride, splits, scale);                             \
    break;
  switch (G) {
    SB_G(1) SB_G(2) SB_G(4) SB_G(5) SB_G(7) SB_G(8)
    default:
      return (int)cudaErrorInvalidValue;
  }
#undef SB_G
  return (int)cudaGetLastError();
}

}  // namespace sb

extern "C" int sb_kv_write(const void* k, const void* v, const int* slots, void* k_cache, void* v_cache, int T,
                           int row_elems, int k_stride, int v_stride, cudaStream_t s) {
  if (T == 0) return 0;
  if (row_elems % 8 != 0 || k_stride % 8 != 0 || v_stride % 8 != 0) return (int)cudaErrorInvalidValue;
  return (int)sb::launch_pdl(sb::kv_write_kernel, dim3(T), dim3(128), 0, s, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                             slots, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, T, row_elems, k_stride, v_stride);
}

// part_o: scratch [B, Hq, splits, D] fp32; part_ml: scratch [B, Hq, splits, 2] fp32.
extern "C" int sb_paged_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                               const int* seq_lens, void* out, float* part_o, float* part_ml, int B, int Hq, int Hkv,
                               int D, int page_size, int max_pages, int q_stride, int out_stride, int splits,
                               float scale, cudaStream_t s) {
  if (B == 0) return 0;
  if (Hq % Hkv != 0) return (int)cudaErrorInvalidValue;
  const int G = Hq / Hkv;
  dim3 grid(B, Hkv, splits);
  int rc;
  if (D == 64)
    rc = sb::launch_decode<64>(G, grid, s, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
                               (const __nv_bfloat16*)v_cache, block_table, seq_lens, part_o, part_ml, Hq, Hkv, page_size,
                               max_pages, q_stride, splits, scale);
  else if (D == 128)
    rc = sb::launch_decode<128>(G, grid, s, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache,
                                (const __nv_bfloat16*)v_cache, block_table, seq_lens, part_o, part_ml, Hq, Hkv, page_size,
                                max_pages, q_stride, splits, scale);
  else
    return (int)cudaErrorInvalidValue;
  if (rc != 0) return rc;
  sb::decode_combine_kernel<<<B * Hq, 64, 0, s>>>(part_o, part_ml, (__nv_bfloat16*)out, D, splits, out_stride, Hq);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- decode step state
// Device-owned per-slot decode state (ids, pos, out_pos) lets consecutive decode steps be launched
// without a host round trip: the sampled token becomes the next input on the device. The host owns
// the block table, the active mask and "init" records for slots that start decoding this step.
namespace sb {

__global__ void decode_prepare_kernel(int* __restrict__ ids, int* __restrict__ pos, int* __restrict__ out_pos,
                                      const int* __restrict__ init_mask, const int* __restrict__ init_ids,
                                      const int* __restrict__ init_pos, const int* __restrict__ init_out_pos,
                                      const int* __restrict__ active, const int* __restrict__ block_table,
                                      int* __restrict__ ids_eff, int* __restrict__ pos_eff, int* __restrict__ seq_lens,
                                      int* __restrict__ slots, int B, int page_size, int max_pages) {
  pdl_wait();  // inputs come from the previous kernel in the stream
  pdl_launch_dependents();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  if (init_mask[b]) {
    ids[b] = init_ids[b];
    pos[b] = init_pos[b];
    out_pos[b] = init_out_pos[b];
  }
  if (active[b]) {
    const int p = pos[b];
    ids_eff[b] = ids[b];
    pos_eff[b] = p;
    seq_lens[b] = p + 1;
    slots[b] = block_table[static_cast<size_t>(b) * max_pages + p / page_size] * page_size + p % page_size;
  } else {  // idle slot: one dummy token whose KV lands in the reserved scratch page 0
    ids_eff[b] = 0;
    pos_eff[b] = 0;
    seq_lens[b] = 1;
    slots[b] = b % page_size;
  }
}

__global__ void decode_advance_kernel(int* __restrict__ ids, int* __restrict__ pos, int* __restrict__ out_pos,
                                      const int* __restrict__ active, const int* __restrict__ sampled, int B) {
  pdl_wait();  // inputs come from the previous kernel in the stream
  pdl_launch_dependents();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B || !active[b]) return;
  ids[b] = sampled[b];
  pos[b] += 1;
  out_pos[b] += 1;
}

}  // namespace sb

extern "C" int sb_decode_prepare(int* ids, int* pos, int* out_pos, const int* init_mask, const int* init_ids,
                                 const int* init_pos, const int* init_out_pos, const int* active, const int* block_table,
                                 int* ids_eff, int* pos_eff, int* seq_lens, int* slots, int B, int page_size,
                                 int max_pages, cudaStream_t s) {
  if (B == 0) return 0;
  return (int)sb::launch_pdl(sb::decode_prepare_kernel, dim3((B + 127) / 128), dim3(128), 0, s, ids, pos, out_pos, init_mask,
                             init_ids, init_pos, init_out_pos, active, block_table, ids_eff, pos_eff, seq_lens, slots, B,
                             page_size, max_pages);
}

extern "C" int sb_decode_advance(int* ids, int* pos, int* out_pos, const int* active, const int* sampled, int B,
                                 cudaStream_t s) {
  if (B == 0) return 0;
  return (int)sb::launch_pdl(sb::decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, s, ids, pos, out_pos, active,
                             sampled, B);
}
