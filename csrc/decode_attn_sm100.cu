// Paged decode attention on the 5th-gen tensor cores (sm_100a): one query token per request, GQA.
//
// Decode attention is bound by streaming the KV cache once, so the kernel is a TMA pipeline with the two small
// contractions on tcgen05 and only the softmax on the CUDA cores:
//
//   per 128-token tile of one (request, kv head, split):
//     TMA      V tile and K tile [128 tok, D] from the paged cache (one box per page) -> smem, 128B swizzle
//     tcgen05  S^T[128 tok, 16]  = K · Q^T          A = K tile (K-major), B = the G <= 16 query heads of this kv head
//     threads  one token per thread: tcgen05.ld its 16 scores, tile max per head, exp, P^T -> smem (bf16, 4 KB)
//     tcgen05  O^T[128(D used), 16] = V^T · P^T     A = V tile read MN-major, B = P^T (K-major)
//     threads  one output dim per thread: tcgen05.ld its 16 values, online-softmax merge into registers
//
//   S^T and P^T are double-buffered: K·Q^T of tile i+1 is issued before the softmax of tile i starts and V^T·P^T of
//   tile i-1 is merged underneath it, so the tensor pipe's latency is off the critical path; three
//   smem stages keep the next tiles' K/V in flight; ~107 KB of smem and 128 TMEM columns per CTA let two CTAs share
//   an SM (D = 64). For D = 64 the V^T operand needs 128 rows: its upper half is pointed at the K tile that follows V in the
//   stage; those 64 accumulator rows are never read.
//   Grid = (B, Hkv, splits); with splits > 1 partial (o, m, l) go to a workspace and a small combine kernel finishes.
//   Every mbarrier wait is bounded (2 s): on expiry the CTA records a status word, skips its output, lets in-flight
//   copies land, frees its TMEM and returns.
//
// Cache layout: k_cache / v_cache = [num_slots, Hkv, D] bf16, slot = page * page_size + offset;
// block_table[b, i] = page id of the i-th page of request b. page_size must be 16, 32, 64 or 128.
#include "common.cuh"

namespace sb {

constexpr int DA_TILE = 128;  // tokens per tile = TMEM lanes = threads
constexpr int DA_THREADS = 128;
constexpr int DA_STAGES = 3;  // K is fetched three tiles ahead, V two: enough bytes in flight to cover HBM latency
constexpr int DA_BT_CACHE = 256;  // block-table entries of this CTA's token range kept in shared memory
constexpr int DA_MAXG = 16;  // N of both MMAs

template <int D>
struct DecSmem {
  static constexpr int NCH = D / 64;                     // 128-byte chunks of the head dim
  static constexpr int KV_TILE = DA_TILE * 128 * NCH;    // bytes of one K (or V) tile
  static constexpr int STAGE = 2 * KV_TILE;              // V then K
  static constexpr int P_BYTES = 2 * DA_MAXG * 128;      // P^T [16 heads, 2 chunks of 64 tokens] bf16, K-major
  static constexpr int Q_BYTES = DA_MAXG * 128 * NCH;    // [16 heads, D] bf16, K-major
  static constexpr int BAR_BYTES = 128;
  static constexpr int TOTAL = DA_STAGES * STAGE + 2 * P_BYTES + Q_BYTES + BAR_BYTES + 1024;  // +1024: manual alignment
  static constexpr int TMEM_COLS = 128;                  // S0 @0, S1 @32, O^T @64 (16 used of each 32)
};

// One-instruction warp maximum (sm_100a: redux.sync on f32).
__device__ __forceinline__ float warp_max_redux(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

template <int D, int G>
__global__ void __launch_bounds__(DA_THREADS)
decode_attn_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const __nv_bfloat16* __restrict__ q, const int* __restrict__ block_table,
                   const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                   float* __restrict__ part_ml, int Hq, int Hkv, int page_size, int page_shift, int max_pages,
                   int q_stride, int out_stride, int splits, float scale, int* status) {
  using S = DecSmem<D>;
  constexpr int NCH = S::NCH;
  static_assert(G <= DA_MAXG, "at most 16 query heads per kv head");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sKV = smem;
  uint8_t* sP = smem + DA_STAGES * S::STAGE;
  uint8_t* sQ = sP + 2 * S::P_BYTES;
  uint64_t* full_k = reinterpret_cast<uint64_t*>(sQ + S::Q_BYTES);
  uint64_t* full_v = full_k + DA_STAGES;
  uint64_t* bar_s = full_v + DA_STAGES;
  uint64_t* bar_o = bar_s + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_o + 1);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ __align__(16) float red_m[2][DA_MAXG][4];  // [S buffer][head][warp]: one 16-byte read per head
  __shared__ float red_l[4][DA_MAXG];
  __shared__ int bt_s[DA_BT_CACHE];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float scale_log2 = scale * 1.4426950408889634f;  // scores live in the log2 domain: exp(x) = 2^(x log2 e)
  const int b = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z;

  if (tid == 0) {
    for (int s = 0; s < DA_STAGES; ++s) {
      mbar_init(&full_k[s], 1);
      mbar_init(&full_v[s], 1);
    }
    mbar_init(&bar_s[0], 1);
    mbar_init(&bar_s[1], 1);
    mbar_init(bar_o, 1);
    *cta_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, S::TMEM_COLS);
    tmem_relinquish();
  }
  // P^T starts as zeros: rows >= G stay zero for the whole kernel, rows < G are rewritten every tile.
  for (int i = tid; i < 2 * S::P_BYTES / 16; i += DA_THREADS) reinterpret_cast<uint4*>(sP)[i] = make_uint4(0, 0, 0, 0);
  // Up to here nothing depended on the previous kernel (barriers, TMEM, the zero fill); the rest reads its outputs.
  pdl_wait();
  pdl_launch_dependents();
  const int len = seq_lens[b];
  const int per_split = ((len + splits - 1) / splits + DA_TILE - 1) & ~(DA_TILE - 1);
  const int t_begin = sp * per_split;
  const int t_end = min(len, t_begin + per_split);
  const int ntiles = t_end > t_begin ? (t_end - t_begin + DA_TILE - 1) / DA_TILE : 0;
  const int* bt_row = block_table + static_cast<size_t>(b) * max_pages;
  // one coalesced read of the page ids this CTA will need, so that issuing a tile's copies does not wait on them
  const int my_pages = t_end > t_begin ? ((t_end - t_begin + page_size - 1) >> page_shift) : 0;
  for (int i = tid; i < min(my_pages, DA_BT_CACHE); i += DA_THREADS) bt_s[i] = bt_row[(t_begin >> page_shift) + i];
  // Q rows (unscaled bf16; the scale is applied to the fp32 scores) in the canonical K-major 128B-swizzle layout:
  // 16-byte chunk j of row r sits at chunk position j ^ (r % 8).
  for (int i = tid; i < DA_MAXG * NCH * 8; i += DA_THREADS) {
    const int r = i / (NCH * 8), c = (i / 8) % NCH, j = i % 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < G)
      v = *reinterpret_cast<const uint4*>(q + static_cast<size_t>(b) * q_stride + static_cast<size_t>(kvh * G + r) * D +
                                          c * 64 + j * 8);
    *reinterpret_cast<uint4*>(sQ + c * (DA_MAXG * 128) + r * 128 + ((j ^ (r & 7)) << 4)) = v;
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 64;

  // warp 0, all lanes: start the copies of the K (or V) half of tile i. Lane p fetches the block-table entry of page p
  // and issues that page's boxes (one per 64-wide chunk of the head dim), so the table reads overlap. K and V have
  // separate barriers because their buffers become free at different times: K once S^T of the tile two back is done,
  // V once that tile's O^T is done. With three stages K runs three tiles ahead of the softmax and V two.
  auto issue_half = [&](int i, bool is_k) {
    const int s = i % DA_STAGES;
    const int t0 = t_begin + i * DA_TILE;
    const int valid = min(DA_TILE, t_end - t0);
    const int npages = (valid + page_size - 1) >> page_shift;
    uint8_t* dst = sKV + s * S::STAGE + (is_k ? S::KV_TILE : 0);
    uint64_t* bar = is_k ? &full_k[s] : &full_v[s];
    if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(npages * page_size * 128 * NCH));
    __syncwarp();
    if (lane < npages) {
      const int pi = ((t0 - t_begin) >> page_shift) + lane;  // page index within this CTA's range
      const int slot0 = (pi < DA_BT_CACHE ? bt_s[pi] : bt_row[(t_begin >> page_shift) + pi]) * page_size;
#pragma unroll
      for (int c = 0; c < NCH; ++c)
        tma_load_3d(dst + c * (DA_TILE * 128) + lane * page_size * 128, is_k ? &tmK : &tmV, bar, c * 64, kvh, slot0);
    }
    __syncwarp();
  };
  // thread 0 only: S^T[128 tok, 16] = K_tile · Q^T into S buffer (i & 1)
  auto issue_s_mma = [&](int i) {
    constexpr uint32_t idesc = make_idesc(DA_TILE, DA_MAXG, 1, 1, 0, 0);
    const uint32_t k_addr = smem_u32(sKV + (i % DA_STAGES) * S::STAGE + S::KV_TILE);
    const uint32_t q_addr = smem_u32(sQ);
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_f16(tmem_base + (i & 1) * 32, make_smem_desc(k_addr + c * (DA_TILE * 128) + k * 32, 16, 1024, UMMA_SWIZZLE_128B),
                 make_smem_desc(q_addr + c * (DA_MAXG * 128) + k * 32, 16, 1024, UMMA_SWIZZLE_128B), idesc,
                 (c | k) != 0 ? 1u : 0u);
    umma_commit(&bar_s[i & 1]);
  };
  // thread 0 only: O^T[128, 16] = V_tile^T · P^T (fresh accumulator every tile; the merge happens in registers).
  // A is the V tile read MN-major: 64-wide chunks of the head dim are DA_TILE*128 bytes apart; with D = 64 the second
  // chunk is the K tile, whose 64 product rows are ignored.
  auto issue_o_mma = [&](int i) {
    constexpr uint32_t idesc = make_idesc(128, DA_MAXG, 1, 1, 1, 0);
    const uint32_t v_addr = smem_u32(sKV + (i % DA_STAGES) * S::STAGE);
    const uint32_t p_addr = smem_u32(sP + (i & 1) * S::P_BYTES);
#pragma unroll
    for (int kc = 0; kc < 2; ++kc)
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_f16(tmem_o, make_smem_desc(v_addr + (kc * 4 + k) * 2048, DA_TILE * 128, 1024, UMMA_SWIZZLE_128B),
                 make_smem_desc(p_addr + kc * (DA_MAXG * 128) + k * 32, 16, 1024, UMMA_SWIZZLE_128B), idesc,
                 (kc | k) != 0 ? 1u : 0u);
    umma_commit(bar_o);
  };

  bool ok = true;
  if (warp == 0 && ntiles > 0) {
    for (int t = 0; t < min(ntiles, DA_STAGES); ++t) {
      issue_half(t, true);
      issue_half(t, false);
    }
    if (lane == 0) {
      ok = mbar_wait(&full_k[0], 0, cta_abort, status, ERR_WAIT_FULL);
      if (ok) {
        tc_fence_after();
        issue_s_mma(0);
      }
    }
    __syncwarp();
  }

  // Running softmax state. Thread d (< D) owns output dim d of all G heads. The denominator is kept per thread (each
  // thread sums the p of its own tokens, rescaled like the accumulator) and reduced once at the end. `keep`/`gain`
  // are the factors a tile's merge applies: acc = acc * keep + o_tile * gain. A tile is merged one iteration after
  // its softmax, underneath the next tile's, so the tensor pipe's latency stays off the critical path.
  float acc[G], m_thr[G], l_thr[G], keep_prev[G], gain_prev[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    acc[g] = 0.f;
    m_thr[g] = -INFINITY;
    l_thr[g] = 0.f;
    keep_prev[g] = 1.f;
    gain_prev[g] = 0.f;
  }
  const bool merges = tid < D;  // warp-uniform: D is 64 or 128
  // merge tile j (O^T is ready once bar_o completes phase j); its V buffer is then free for tile j + DA_STAGES
  auto merge_tile = [&](int j) -> bool {
    bool okm = mbar_wait(bar_o, j & 1, cta_abort, status, ERR_WAIT_TMEM_FULL);
    okm = __all_sync(0xffffffffu, okm);
    tc_fence_after();
    if (okm && merges) {
      uint32_t r[32];
      tmem_ld_32x32(tmem_o + (static_cast<uint32_t>(warp * 32) << 16), r);
      tmem_ld_wait();
#pragma unroll
      for (int g = 0; g < G; ++g) acc[g] = acc[g] * keep_prev[g] + __uint_as_float(r[g]) * gain_prev[g];
    }
    if (okm && warp == 0 && j + DA_STAGES < ntiles) issue_half(j + DA_STAGES, false);
    return okm;
  };

  for (int i = 0; i < ntiles; ++i) {
    const int s = i % DA_STAGES, par = i & 1;
    const int t0 = t_begin + i * DA_TILE;
    const int valid = min(DA_TILE, t_end - t0);
    // ---- scores of this thread's token (TMEM lane = tid) for the G heads
    if (ok) ok = mbar_wait(&bar_s[par], (i >> 1) & 1, cta_abort, status, ERR_WAIT_TMEM_FULL);
    if (tid == 0 && ok && i + 1 < ntiles) {
      // K·Q^T of the next tile goes to the other S^T buffer now, so it runs underneath this tile's softmax
      if (mbar_wait(&full_k[(i + 1) % DA_STAGES], ((i + 1) / DA_STAGES) & 1, cta_abort, status, ERR_WAIT_FULL)) {
        tc_fence_after();
        issue_s_mma(i + 1);
      } else {
        ok = false;
      }
    }
    ok = __all_sync(0xffffffffu, ok);  // the TMEM load below is warp-collective: take one decision per warp
    tc_fence_after();
    float sc[G];
    {
      uint32_t r[32];
      if (ok) {
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + par * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int g = 0; g < 32; ++g) r[g] = 0;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) sc[g] = (tid < valid) ? __uint_as_float(r[g]) * scale_log2 : -INFINITY;
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float wm = warp_max_redux(sc[g]);
      if (lane == 0) red_m[par][g][warp] = wm;
    }
    ok = __syncthreads_and(ok);  // (A) tile maxima visible; everyone agrees whether to go on
    if (!ok) break;
    // S^T of this tile is complete, so nothing reads its K buffer any more: refill it for the tile two ahead
    if (warp == 0 && i + DA_STAGES < ntiles) issue_half(i + DA_STAGES, true);

    // ---- the previous tile's product is done by now (it was issued before this tile's scores were read): fold it
    //      in, which also frees O^T and the P^T buffer of two tiles ago for reuse below
    if (i > 0) ok = merge_tile(i - 1);

    // ---- p = exp(s - tile max), rounded to bf16 exactly as the tensor core will see it
    const int kc = tid >> 6, col = tid & 63;
    uint8_t* p_col = sP + par * S::P_BYTES + kc * (DA_MAXG * 128) + (col & 7) * 2;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float4 wmx = *reinterpret_cast<const float4*>(red_m[par][g]);
      const float mt = fmaxf(fmaxf(wmx.x, wmx.y), fmaxf(wmx.z, wmx.w));
      const float p = fast_exp2(sc[g] - mt);  // tokens past the end have sc = -inf -> p = 0
      const __nv_bfloat16 pb = __float2bfloat16(p);  // the denominator sums the unrounded p (rounding is unbiased)
      const float nm = fmaxf(m_thr[g], mt);  // the same for every thread of the CTA
      const float keep = fast_exp2(m_thr[g] - nm);  // first tile: 2^(-inf) = 0
      const float gain = fast_exp2(mt - nm);
      l_thr[g] = l_thr[g] * keep + p * gain;
      m_thr[g] = nm;
      keep_prev[g] = keep;
      gain_prev[g] = gain;
      *reinterpret_cast<__nv_bfloat16*>(p_col + g * 128 + (((col >> 3) ^ (g & 7)) << 4)) = pb;
    }
    if (valid < DA_TILE) {
      // Last tile: rows past the end of the sequence hold whatever the cache (or an older tile) left there.
      // Their p is 0, but 0 x NaN would poison O, so the V rows are cleared. Every thread observes the copy's
      // barrier first so that its plain stores are ordered after the TMA writes.
      if (ok) ok = mbar_wait(&full_v[s], (i / DA_STAGES) & 1, cta_abort, status, ERR_WAIT_FULL);
      if (ok && tid >= valid) {
        uint8_t* vrow = sKV + s * S::STAGE + tid * 128;
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
          for (int j = 0; j < 8; ++j)
            reinterpret_cast<uint4*>(vrow + c * (DA_TILE * 128))[j] = make_uint4(0, 0, 0, 0);
      }
    }
    fence_proxy_async();  // P^T (and cleared V rows) -> visible to the tensor core's async proxy
    tc_fence_before();    // ... and this thread's TMEM reads (scores, previous O^T) are ordered before the next MMAs
    ok = __syncthreads_and(ok);  // (B)
    if (!ok) break;

    if (tid == 0) {
      if (mbar_wait(&full_v[s], (i / DA_STAGES) & 1, cta_abort, status, ERR_WAIT_FULL)) {
        tc_fence_after();
        issue_o_mma(i);
      } else {
        ok = false;
      }
    }
    __syncwarp();
  }
  ok = __syncthreads_and(ok);  // one decision for the whole CTA: the merges below contain warp-collective steps
  if (ok && ntiles > 0) ok = merge_tile(ntiles - 1);

  // ---- denominators: one block reduction per head (all l_thr[g] refer to the same final maximum)
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float ws = warp_sum(l_thr[g]);
    if (lane == 0) red_l[warp][g] = ws;
  }
  const bool all_ok = __syncthreads_and(ok) && (*cta_abort == 0);
  // ---- output: thread d writes dim d of each head (consecutive threads -> consecutive addresses)
  if (all_ok && merges) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float l_run = red_l[0][g] + red_l[1][g] + red_l[2][g] + red_l[3][g];
      const int h = kvh * G + g;
      if (splits == 1) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        out[static_cast<size_t>(b) * out_stride + static_cast<size_t>(h) * D + tid] = __float2bfloat16(acc[g] * inv);
      } else {
        const size_t base = (static_cast<size_t>(b) * Hq + h) * splits + sp;
        part_o[base * D + tid] = acc[g];
        if (tid == 0) {
          part_ml[base * 2 + 0] = m_thr[g] * 0.6931471805599453f;  // back to the natural-log domain
          part_ml[base * 2 + 1] = l_run;
        }
      }
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    // give copies that are still in flight a bounded time to land before the shared memory goes away
    const unsigned long long t_a = globaltimer_ns();
    while (globaltimer_ns() - t_a < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem_base, S::TMEM_COLS);
}

// out[b, h, :] = sum_s o_s exp(m_s - M) / sum_s l_s exp(m_s - M) over the splits of one (request, head).
__global__ void decode_attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           __nv_bfloat16* __restrict__ out, int D, int splits, int out_stride, int Hq) {
  pdl_wait();
  pdl_launch_dependents();
  const int bh = blockIdx.x, b = bh / Hq, h = bh % Hq;
  const float* ml = part_ml + static_cast<size_t>(bh) * splits * 2;
  float gm = -INFINITY;
  for (int s = 0; s < splits; ++s) gm = fmaxf(gm, ml[2 * s]);
  float gl = 0.f;
  for (int s = 0; s < splits; ++s)
    if (ml[2 * s] != -INFINITY) gl += ml[2 * s + 1] * __expf(ml[2 * s] - gm);
  const float inv = gl > 0.f ? 1.f / gl : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < splits; ++s)
      if (ml[2 * s] != -INFINITY) o += part_o[(static_cast<size_t>(bh) * splits + s) * D + d] * __expf(ml[2 * s] - gm);
    out[static_cast<size_t>(b) * out_stride + static_cast<size_t>(h) * D + d] = __float2bfloat16(o * inv);
  }
}

// [num_slots, Hkv, D] bf16 cache as a 3-D tensor map; box = one page of one head, 64 elements (128 B) wide.
static CUtensorMap make_cache_tmap(const void* base, int num_slots, int Hkv, int D, int page_size) {
  CUtensorMap m;
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)Hkv, (cuuint64_t)num_slots};
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)Hkv * D * 2};
  cuuint32_t box[3] = {64, 1, (cuuint32_t)page_size};
  cuuint32_t estr[3] = {1, 1, 1};
  static thread_local bool ctx_bound = false;  // the encoder needs the primary context current on this thread
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) ctx_bound = true;
  }
  CUresult r = get_encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw std::runtime_error("cuTensorMapEncodeTiled (kv cache) failed: " + std::to_string(int(r)) + " slots=" +
                             std::to_string(num_slots) + " Hkv=" + std::to_string(Hkv) + " D=" + std::to_string(D));
  return m;
}

template <int D, int G>
static int launch_decode_attn(dim3 grid, cudaStream_t s, const CUtensorMap& tk, const CUtensorMap& tv, const __nv_bfloat16* q,
                              const int* bt, const int* sl, __nv_bfloat16* out, float* po, float* pml, int Hq, int Hkv,
                              int page_size, int page_shift, int max_pages, int q_stride, int out_stride, int splits,
                              float scale, int* status) {
  auto kern = decode_attn_kernel<D, G>;
  if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), DecSmem<D>::TOTAL); e != cudaSuccess) return (int)e;
  return (int)launch_pdl(kern, grid, dim3(DA_THREADS), DecSmem<D>::TOTAL, s, tk, tv, q, bt, sl, out, po, pml, Hq, Hkv,
                         page_size, page_shift, max_pages, q_stride, out_stride, splits, scale, status);
}

}  // namespace sb

// Returns 0, a cudaError_t value, or -1 when the shape is outside what this kernel covers (the caller then uses
// the CUDA-core kernel sb_paged_decode). part_o / part_ml: workspaces [B, Hq, splits, D] / [B, Hq, splits, 2] fp32,
// only touched when splits > 1.
extern "C" int sb_paged_decode_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                  const int* seq_lens, void* out, float* part_o, float* part_ml, int B, int Hq, int Hkv,
                                  int D, int page_size, int max_pages, int num_slots, int q_stride, int out_stride,
                                  int splits, float scale, int* status, cudaStream_t s) {
  using bf16 = __nv_bfloat16;
  if (B == 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0 || (D != 64 && D != 128)) return -1;
  const int G = Hq / Hkv;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  if ((1 << page_shift) != page_size || page_size < 16 || page_size > 128) return -1;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (q_stride & 7) || (reinterpret_cast<uintptr_t>(out) & 15) || (out_stride & 7) ||
      (reinterpret_cast<uintptr_t>(k_cache) & 127) || (reinterpret_cast<uintptr_t>(v_cache) & 127))
    return -1;
  try {
    const CUtensorMap tk = sb::make_cache_tmap(k_cache, num_slots, Hkv, D, page_size);
    const CUtensorMap tv = sb::make_cache_tmap(v_cache, num_slots, Hkv, D, page_size);
    dim3 grid(B, Hkv, splits);
    int rc = -1;
#define SB_DA(DV, GV)                                                                                                  \
  if (D == DV && G == GV)                                                                                              \
    rc = sb::launch_decode_attn<DV, GV>(grid, s, tk, tv, (const bf16*)q, block_table, seq_lens, (bf16*)out, part_o, part_ml, \
                                        Hq, Hkv, page_size, page_shift, max_pages, q_stride, out_stride, splits, scale, status);
    SB_DA(64, 1) SB_DA(64, 2) SB_DA(64, 4) SB_DA(64, 5) SB_DA(64, 6) SB_DA(64, 7) SB_DA(64, 8) SB_DA(64, 16)
    SB_DA(128, 1) SB_DA(128, 2) SB_DA(128, 4) SB_DA(128, 5) SB_DA(128, 6) SB_DA(128, 7) SB_DA(128, 8) SB_DA(128, 16)
#undef SB_DA
    if (rc != 0) return rc;
    if (splits > 1)
      return (int)sb::launch_pdl(sb::decode_attn_combine_kernel, dim3(B * Hq), dim3(64), 0, s, part_o, part_ml, (bf16*)out, D,
                                 splits, out_stride, Hq);
    return (int)cudaGetLastError();
  } catch (const std::exception& e) {
    sb::set_last_error(e.what());
    return (int)cudaErrorInvalidValue;
  }
}
