// Memory-bound fused ops for sm_100a: (residual add +) RMSNorm fwd/bwd, per-head
// QK-RMSNorm + RoPE fwd/bwd on packed [T, H, D] tensors, SwiGLU fwd/bwd, embedding
// gather / scatter-add. One pass over HBM per tensor, 16-byte vector accesses,
// fp32 math. The same kernels serve the trainer and the rollout engine so both
// sides round identically (norm is computed from the un-rounded fp32 residual sum).
#include "common.cuh"

namespace sb {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_VEC = 4;  // up to 4 x 8 bf16 per thread cached in registers -> H <= 8192

struct bf16x8 {
  uint4 u;
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ void load8(const float* p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// y = rmsnorm(x (+ res)) * w ; optionally res_out = x + res (bf16) ; rstd[T] saved for backward.
// H % 8 == 0, H <= 8192. grid = T rows. XT = bf16, or float when x is the fp32 sum left by a split-K projection.
template <typename XT>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const XT* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float scratch[32];
  pdl_wait();  // inputs come from the previous kernel in the stream
  pdl_launch_dependents();
  const size_t row = blockIdx.x;
  const int nvec = H >> 3;
  float v[NORM_MAX_VEC][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NORM_MAX_VEC; ++j) {
    const int c = threadIdx.x + j * NORM_THREADS;
    if (c < nvec) {
      load8(x + row * H + c * 8, v[j]);
      if (res != nullptr) {
        float r[8];
        load8(res + row * H + c * 8, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[j][i] += r[i];
      }
      if (res_out != nullptr) store8(res_out + row * H + c * 8, v[j]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[j][i] * v[j][i];
    }
  }
  ss = block_sum<NORM_THREADS>(ss, scratch);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
  for (int j = 0; j < NORM_MAX_VEC; ++j) {
    const int c = threadIdx.x + j * NORM_THREADS;
    if (c < nvec) {
      float g[8], o[8];
      load8(w + c * 8, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = v[j][i] * rstd * g[i];
      store8(y + row * H + c * 8, o);
    }
  }
}

// Backward of y = rmsnorm(h) * w for a strip of rows per CTA (h = the summed residual input).
//   dh = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres_in)
//   dw_partial[cta, :] = sum over the CTA's rows of dy * xhat
// dw_partial is scratch of shape [gridDim.x, H] fp32, reduced by rmsnorm_dw_reduce_kernel.
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dh,
                   float* __restrict__ dw_partial, int T, int H) {
  __shared__ float scratch[32];
  const int nvec = H >> 3;
  float dwacc[NORM_MAX_VEC][8];
  float g[NORM_MAX_VEC][8];
#pragma unroll
  for (int j = 0; j < NORM_MAX_VEC; ++j) {
    const int c = threadIdx.x + j * NORM_THREADS;
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[j][i] = 0.f;
    if (c < nvec) load8(w + c * 8, g[j]);
  }
  for (size_t row = blockIdx.x; row < static_cast<size_t>(T); row += gridDim.x) {
    const float rs = rstd[row];
    float xh[NORM_MAX_VEC][8], dyw[NORM_MAX_VEC][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_MAX_VEC; ++j) {
      const int c = threadIdx.x + j * NORM_THREADS;
      if (c < nvec) {
        float a[8], b[8];
        load8(dy + row * H + c * 8, a);
        load8(h + row * H + c * 8, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[j][i] = b[i] * rs;
          dwacc[j][i] += a[i] * xh[j][i];
          dyw[j][i] = a[i] * g[j][i];
          dot += dyw[j][i] * xh[j][i];
        }
      }
    }
    dot = block_sum<NORM_THREADS>(dot, scratch) / H;
#pragma unroll
    for (int j = 0; j < NORM_MAX_VEC; ++j) {
      const int c = threadIdx.x + j * NORM_THREADS;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rs * (dyw[j][i] - xh[j][i] * dot);
        if (dres_in != nullptr) {
          float r[8];
          load8(dres_in + row * H + c * 8, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += r[i];
        }
        store8(dh + row * H + c * 8, o);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NORM_MAX_VEC; ++j) {
    const int c = threadIdx.x + j * NORM_THREADS;
    if (c < nvec) {
      float4* dst = reinterpret_cast<float4*>(dw_partial + static_cast<size_t>(blockIdx.x) * H + c * 8);
      dst[0] = make_float4(dwacc[j][0], dwacc[j][1], dwacc[j][2], dwacc[j][3]);
      dst[1] = make_float4(dwacc[j][4], dwacc[j][5], dwacc[j][6], dwacc[j][7]);
    }
  }
}

// dw[c] (+)= sum_p dw_partial[p, c]
__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ part, float* __restrict__ dw, int P, int H,
                                         int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += part[static_cast<size_t>(p) * H + c];
  dw[c] = accumulate ? dw[c] + s : s;
}

// Same backward for rows of at most 1024 elements: one WARP per row, so a row costs one shuffle reduction and no
// block barrier, and every warp keeps 2 * VPL independent 16-byte loads in flight. Lane l owns the 8-element
// vectors l, l + 32, ... (VPL of them). The per-column dw sums of the CTA's 8 warps are combined in shared memory in
// warp order (deterministic) and written as one partial row per CTA.
template <int VPL>
__global__ void __launch_bounds__(NORM_THREADS, 2)
rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                        const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dh,
                        float* __restrict__ dw_partial, int T, int H) {
  constexpr int WARPS = NORM_THREADS / 32;
  __shared__ float dw_sh[32 * VPL * 8];
  const int nvec = H >> 3, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_h = 1.f / static_cast<float>(H);
  uint4 gw[VPL];  // the weight stays packed (4 registers per vector) and is unpacked where it is used
  float dwacc[VPL][8];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int c = lane + 32 * j;
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[j][i] = 0.f;
    gw[j] = c < nvec ? *reinterpret_cast<const uint4*>(w + c * 8) : make_uint4(0, 0, 0, 0);
  }
  for (size_t row = static_cast<size_t>(blockIdx.x) * WARPS + warp; row < static_cast<size_t>(T);
       row += static_cast<size_t>(gridDim.x) * WARPS) {
    const float rs = rstd[row];
    uint4 ra[VPL], rb[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) {  // all loads of the row first
      const int c = lane + 32 * j;
      ra[j] = rb[j] = make_uint4(0, 0, 0, 0);
      if (c < nvec) {
        ra[j] = *reinterpret_cast<const uint4*>(dy + row * H + c * 8);
        rb[j] = *reinterpret_cast<const uint4*>(h + row * H + c * 8);
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      float a[8], b[8], g[8];
      unpack8(ra[j], a);
      unpack8(rb[j], b);
      unpack8(gw[j], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = b[i] * rs;
        dwacc[j][i] += a[i] * xh;
        dot += a[i] * g[i] * xh;
      }
    }
    dot = warp_sum(dot) * inv_h;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int c = lane + 32 * j;
      if (c < nvec) {
        float a[8], b[8], r[8], g[8], o[8];
        unpack8(ra[j], a);
        unpack8(rb[j], b);
        unpack8(dres_in != nullptr ? *reinterpret_cast<const uint4*>(dres_in + row * H + c * 8) : make_uint4(0, 0, 0, 0), r);
        unpack8(gw[j], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rs * (a[i] * g[i] - b[i] * rs * dot) + r[i];
        store8(dh + row * H + c * 8, o);
      }
    }
  }
  for (int turn = 0; turn < WARPS; ++turn) {
    if (warp == turn) {
#pragma unroll
      for (int j = 0; j < VPL; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float* slot = &dw_sh[(lane + 32 * j) * 8 + i];
          *slot = turn == 0 ? dwacc[j][i] : *slot + dwacc[j][i];
        }
    }
    __syncthreads();
  }
  for (int c = threadIdx.x; c < H; c += NORM_THREADS) dw_partial[static_cast<size_t>(blockIdx.x) * H + c] = dw_sh[c];
}

// Both backward entry points launch through here: the warp-per-row kernel up to H = 1024, the block-per-row
// kernel above that, then the reduction of the per-CTA dw partials.
static cudaError_t launch_rmsnorm_bwd(const __nv_bfloat16* dy, const __nv_bfloat16* h, const __nv_bfloat16* w,
                                      const float* rstd, const __nv_bfloat16* dres_in, __nv_bfloat16* dh,
                                      float* dw_partial, float* dw, int T, int H, int num_ctas, int accumulate_dw,
                                      cudaStream_t s) {
  const int nvec = H >> 3;
  if (nvec <= 32)
    rmsnorm_bwd_warp_kernel<1><<<num_ctas, NORM_THREADS, 0, s>>>(dy, h, w, rstd, dres_in, dh, dw_partial, T, H);
  else if (nvec <= 64)
    rmsnorm_bwd_warp_kernel<2><<<num_ctas, NORM_THREADS, 0, s>>>(dy, h, w, rstd, dres_in, dh, dw_partial, T, H);
  else if (nvec <= 128)
    rmsnorm_bwd_warp_kernel<4><<<num_ctas, NORM_THREADS, 0, s>>>(dy, h, w, rstd, dres_in, dh, dw_partial, T, H);
  else
    rmsnorm_bwd_kernel<<<num_ctas, NORM_THREADS, 0, s>>>(dy, h, w, rstd, dres_in, dh, dw_partial, T, H);
  rmsnorm_dw_reduce_kernel<<<(H + 255) / 256, 256, 0, s>>>(dw_partial, dw, num_ctas, H, accumulate_dw);
  return cudaGetLastError();
}

// ---------------------------------------------------------------- QK-norm + RoPE
// x: [T, heads_total, D] packed (q heads then k heads then v heads in one qkv row is fine:
// `row_stride` is the element pitch of a token, `head0` the first head to process, `nheads`
// how many). One warp per (token, head). Rotate-half convention:
//   o[i] = a[i] cos - a[i+D/2] sin ; o[i+D/2] = a[i+D/2] cos + a[i] sin
// with a = x or rmsnorm_D(x) * nw when nw != nullptr. cos/sin table: [max_pos, D/2] fp32.
// `sign` = +1 forward rotation, -1 inverse rotation (backward of RoPE).
template <int D>
__global__ void __launch_bounds__(128)
rope_kernel(const __nv_bfloat16* x, __nv_bfloat16* out /* may alias x: a warp reads its head fully before writing */,
            const int* __restrict__ pos,
            const float* __restrict__ cos_sin, const __nv_bfloat16* __restrict__ nw, float* __restrict__ rstd_out,
            int T, int nheads, int head0, int in_stride, int out_stride, float eps, float sign) {
  constexpr int PER = D / 64;  // each lane handles PER pairs (i, i + D/2) ... D/2 / 32 lanes
  pdl_wait();  // inputs come from the previous kernel in the stream
  pdl_launch_dependents();
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_global >= T * nheads) return;
  const int t = warp_global / nheads, hh = warp_global % nheads;
  const __nv_bfloat16* src = x + static_cast<size_t>(t) * in_stride + static_cast<size_t>(head0 + hh) * D;
  __nv_bfloat16* dst = out + static_cast<size_t>(t) * out_stride + static_cast<size_t>(head0 + hh) * D;
  float lo[PER], hi[PER];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = lane + 32 * j;
    lo[j] = __bfloat162float(src[i]);
    hi[j] = __bfloat162float(src[i + D / 2]);
    ss += lo[j] * lo[j] + hi[j] * hi[j];
  }
  if (nw != nullptr) {
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / D + eps);
    if (rstd_out != nullptr && lane == 0) rstd_out[static_cast<size_t>(t) * nheads + hh] = rs;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = lane + 32 * j;
      lo[j] = lo[j] * rs * __bfloat162float(nw[i]);
      hi[j] = hi[j] * rs * __bfloat162float(nw[i + D / 2]);
    }
  }
  const float* cs = cos_sin + static_cast<size_t>(pos[t]) * D;  // [cos(D/2) | sin(D/2)]
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = lane + 32 * j;
    const float c = cs[i], s = sign * cs[D / 2 + i];
    dst[i] = __float2bfloat16(lo[j] * c - hi[j] * s);
    dst[i + D / 2] = __float2bfloat16(hi[j] * c + lo[j] * s);
  }
}

// Inference form of the above, fused with the KV-cache write: one launch per layer instead of four. One warp per
// (token, head) of a packed qkv row [T, (Hq + 2 Hkv) * D]:
//   q heads  (per-head RMSNorm +) RoPE in place
//   k heads  the same, written in place (prefill attends over the row itself) and to k_cache[slot[t], head]
//   v heads  copied to v_cache[slot[t], head]
// Caches are [slots, Hkv, D] contiguous; a negative slot skips the cache write (padding rows).
template <int D>
__global__ void __launch_bounds__(128)
rope_kv_write_kernel(__nv_bfloat16* qkv, const int* __restrict__ pos, const float* __restrict__ cos_sin,
                     const __nv_bfloat16* __restrict__ q_nw, const __nv_bfloat16* __restrict__ k_nw,
                     const int* __restrict__ slots, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                     int T, int Hq, int Hkv, int row_stride, float eps) {
  constexpr int PER = D / 64;
  pdl_wait();
  pdl_launch_dependents();
  const int heads = Hq + 2 * Hkv;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_global >= T * heads) return;
  const int t = warp_global / heads, h = warp_global % heads;
  __nv_bfloat16* row = qkv + static_cast<size_t>(t) * row_stride + static_cast<size_t>(h) * D;
  if (h >= Hq + Hkv) {  // v: copy to the cache
    const int slot = slots[t];
    if (slot < 0) return;
    __nv_bfloat16* dst = v_cache + (static_cast<size_t>(slot) * Hkv + (h - Hq - Hkv)) * D;
    const uint32_t* s32 = reinterpret_cast<const uint32_t*>(row);
    uint32_t* d32 = reinterpret_cast<uint32_t*>(dst);
#pragma unroll
    for (int j = 0; j < PER; ++j) d32[lane + 32 * j] = s32[lane + 32 * j];
    return;
  }
  const bool is_k = h >= Hq;
  const __nv_bfloat16* nw = is_k ? k_nw : q_nw;
  float lo[PER], hi[PER];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = lane + 32 * j;
    lo[j] = __bfloat162float(row[i]);
    hi[j] = __bfloat162float(row[i + D / 2]);
    ss += lo[j] * lo[j] + hi[j] * hi[j];
  }
  if (nw != nullptr) {
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / D + eps);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = lane + 32 * j;
      lo[j] = lo[j] * rs * __bfloat162float(nw[i]);
      hi[j] = hi[j] * rs * __bfloat162float(nw[i + D / 2]);
    }
  }
  const float* cs = cos_sin + static_cast<size_t>(pos[t]) * D;  // [cos(D/2) | sin(D/2)]
  const int slot = is_k ? slots[t] : -1;
  __nv_bfloat16* cache = slot >= 0 ? k_cache + (static_cast<size_t>(slot) * Hkv + (h - Hq)) * D : nullptr;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = lane + 32 * j;
    const float c = cs[i], sn = cs[D / 2 + i];
    const __nv_bfloat16 a = __float2bfloat16(lo[j] * c - hi[j] * sn), b = __float2bfloat16(hi[j] * c + lo[j] * sn);
    row[i] = a;
    row[i + D / 2] = b;
    if (cache != nullptr) {
      cache[i] = a;
      cache[i + D / 2] = b;
    }
  }
}

// ---------------------------------------------------------------------- SwiGLU
// gu: [T, 2F] = [gate | up]; act[T, F] = silu(gate) * up
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, size_t T, int F) {
  pdl_wait();  // inputs come from the previous kernel in the stream
  pdl_launch_dependents();
  const size_t nvec = T * (F >> 3);
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < nvec;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = idx / (F >> 3);
    const int c = static_cast<int>(idx % (F >> 3)) * 8;
    float g[8], u[8], o[8];
    load8(gu + t * 2 * F + c, g);
    load8(gu + t * 2 * F + F + c, u);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
    store8(act + t * F + c, o);
  }
}

// dgu = [dact * up * dsilu(gate) | dact * silu(gate)]
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* __restrict__ dgu, size_t T, int F) {
  const size_t nvec = T * (F >> 3);
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < nvec;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = idx / (F >> 3);
    const int c = static_cast<int>(idx % (F >> 3)) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + t * 2 * F + c, g);
    load8(gu + t * 2 * F + F + c, u);
    load8(dact + t * F + c, d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sg = 1.f / (1.f + __expf(-g[i]));
      const float silu = g[i] * sg;
      dg[i] = d[i] * u[i] * (sg + silu * (1.f - sg));
      du[i] = d[i] * silu;
    }
    store8(dgu + t * 2 * F + c, dg);
    store8(dgu + t * 2 * F + F + c, du);
  }
}

// ------------------------------------------------------------------- embedding
__global__ void embedding_fwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int T, int H, int vocab_lo, int vocab_hi) {
  pdl_wait();  // inputs come from the previous kernel in the stream
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool mine = id >= vocab_lo && id < vocab_hi;
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(mine ? id - vocab_lo : 0) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H);
  for (int c = threadIdx.x; c < (H >> 3); c += blockDim.x) dst[c] = mine ? src[c] : make_uint4(0, 0, 0, 0);
}

// dtable[id] += dout[t] in fp32 (atomic; rows with repeated ids collide rarely enough at 150k vocab)
__global__ void embedding_bwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dtable, int T, int H, int vocab_lo, int vocab_hi) {
  const int t = blockIdx.x;
  const int id = ids[t];
  if (id < vocab_lo || id >= vocab_hi) return;
  float* dst = dtable + static_cast<size_t>(id - vocab_lo) * H;
  const __nv_bfloat16* src = dout + static_cast<size_t>(t) * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) atomicAdd(dst + c, __bfloat162float(src[c]));
}

// out = a + b (bf16), 8-wide
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ out, size_t nvec) {
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < nvec;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float x[8], y[8];
    load8(a + idx * 8, x);
    load8(b + idx * 8, y);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] += y[i];
    store8(out + idx * 8, x);
  }
}

}  // namespace sb

using bf16 = __nv_bfloat16;

extern "C" int sb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out, float* rstd,
                              int T, int H, float eps, cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8 != 0 || H > sb::NORM_THREADS * sb::NORM_MAX_VEC * 8) return (int)cudaErrorInvalidValue;
  return (int)sb::launch_pdl(sb::rmsnorm_fwd_kernel<bf16>, dim3(T), dim3(sb::NORM_THREADS), 0, s, (const bf16*)x,
                             (const bf16*)res, (const bf16*)w, (bf16*)y, (bf16*)res_out, rstd, H, eps);
}

// Same, with x in fp32 (res, w, y, res_out stay bf16).
extern "C" int sb_rmsnorm_fwd_f32x(const float* x, const void* res, const void* w, void* y, void* res_out, float* rstd,
                                   int T, int H, float eps, cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8 != 0 || H > sb::NORM_THREADS * sb::NORM_MAX_VEC * 8) return (int)cudaErrorInvalidValue;
  return (int)sb::launch_pdl(sb::rmsnorm_fwd_kernel<float>, dim3(T), dim3(sb::NORM_THREADS), 0, s, x, (const bf16*)res,
                             (const bf16*)w, (bf16*)y, (bf16*)res_out, rstd, H, eps);
}

// dw_partial: scratch [num_ctas, H] fp32 supplied by the caller; dw: [H] fp32.
extern "C" int sb_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres_in,
                              void* dh, float* dw_partial, float* dw, int T, int H, int num_ctas, int accumulate_dw,
                              cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8 != 0 || H > sb::NORM_THREADS * sb::NORM_MAX_VEC * 8) return (int)cudaErrorInvalidValue;
  return (int)sb::launch_rmsnorm_bwd((const bf16*)dy, (const bf16*)h, (const bf16*)w, rstd, (const bf16*)dres_in,
                                     (bf16*)dh, dw_partial, dw, T, H, num_ctas, accumulate_dw, s);
}

extern "C" int sb_rope(const void* x, void* out, const int* pos, const float* cos_sin, const void* nw, float* rstd,
                       int T, int nheads, int head0, int in_stride, int out_stride, int D, float eps, float sign,
                       cudaStream_t s) {
  if (T == 0 || nheads == 0) return 0;
  const long warps = (long)T * nheads;
  const int blocks = (int)((warps * 32 + 127) / 128);
  if (D == 64)
    return (int)sb::launch_pdl(sb::rope_kernel<64>, dim3(blocks), dim3(128), 0, s, (const bf16*)x, (bf16*)out, pos, cos_sin,
                               (const bf16*)nw, rstd, T, nheads, head0, in_stride, out_stride, eps, sign);
  else if (D == 128)
    return (int)sb::launch_pdl(sb::rope_kernel<128>, dim3(blocks), dim3(128), 0, s, (const bf16*)x, (bf16*)out, pos, cos_sin,
                               (const bf16*)nw, rstd, T, nheads, head0, in_stride, out_stride, eps, sign);
  else if (D == 256)
    return (int)sb::launch_pdl(sb::rope_kernel<256>, dim3(blocks), dim3(128), 0, s, (const bf16*)x, (bf16*)out, pos, cos_sin,
                               (const bf16*)nw, rstd, T, nheads, head0, in_stride, out_stride, eps, sign);
  else
    return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

extern "C" int sb_rope_kv_write(void* qkv, const int* pos, const float* cos_sin, const void* q_nw, const void* k_nw,
                                const int* slots, void* k_cache, void* v_cache, int T, int Hq, int Hkv, int D, int row_stride,
                                float eps, cudaStream_t s) {
  if (T == 0) return 0;
  if ((row_stride & 1) || (reinterpret_cast<uintptr_t>(qkv) & 3)) return (int)cudaErrorInvalidValue;
  const long warps = (long)T * (Hq + 2 * Hkv);
  const int blocks = (int)((warps * 32 + 127) / 128);
#define SB_RKW(DV)                                                                                                     \
  if (D == DV)                                                                                                         \
    return (int)sb::launch_pdl(sb::rope_kv_write_kernel<DV>, dim3(blocks), dim3(128), 0, s, (bf16*)qkv, pos, cos_sin,  \
                               (const bf16*)q_nw, (const bf16*)k_nw, slots, (bf16*)k_cache, (bf16*)v_cache, T, Hq, Hkv, \
                               row_stride, eps);
  SB_RKW(64) SB_RKW(128) SB_RKW(256)
#undef SB_RKW
  return (int)cudaErrorInvalidValue;
}

static inline int ew_blocks(size_t n, int threads) {
  size_t b = (n + threads - 1) / threads;
  return (int)(b > 148 * 16 ? 148 * 16 : (b == 0 ? 1 : b));
}

extern "C" int sb_swiglu_fwd(const void* gu, void* act, long T, int F, cudaStream_t s) {
  if (T == 0) return 0;
  if (F % 8 != 0) return (int)cudaErrorInvalidValue;
  return (int)sb::launch_pdl(sb::swiglu_fwd_kernel, dim3(ew_blocks((size_t)T * (F / 8), 256)), dim3(256), 0, s, (const bf16*)gu,
                             (bf16*)act, (size_t)T, F);
}

extern "C" int sb_swiglu_bwd(const void* gu, const void* dact, void* dgu, long T, int F, cudaStream_t s) {
  if (T == 0) return 0;
  if (F % 8 != 0) return (int)cudaErrorInvalidValue;
  sb::swiglu_bwd_kernel<<<ew_blocks((size_t)T * (F / 8), 256), 256, 0, s>>>((const bf16*)gu, (const bf16*)dact,
                                                                             (bf16*)dgu, (size_t)T, F);
  return (int)cudaGetLastError();
}

extern "C" int sb_embedding_fwd(const int* ids, const void* table, void* out, int T, int H, int vlo, int vhi,
                                cudaStream_t s) {
  if (T == 0) return 0;
  return (int)sb::launch_pdl(sb::embedding_fwd_kernel, dim3(T), dim3(128), 0, s, ids, (const bf16*)table, (bf16*)out, T, H,
                             vlo, vhi);
}

extern "C" int sb_embedding_bwd(const int* ids, const void* dout, float* dtable, int T, int H, int vlo, int vhi,
                                cudaStream_t s) {
  if (T == 0) return 0;
  sb::embedding_bwd_kernel<<<T, 256, 0, s>>>(ids, (const bf16*)dout, dtable, T, H, vlo, vhi);
  return (int)cudaGetLastError();
}

extern "C" int sb_add_bf16(const void* a, const void* b, void* out, long n, cudaStream_t s) {
  if (n == 0) return 0;
  if (n % 8 != 0) return (int)cudaErrorInvalidValue;
  sb::add_bf16_kernel<<<ew_blocks((size_t)n / 8, 256), 256, 0, s>>>((const bf16*)a, (const bf16*)b, (bf16*)out,
                                                                    (size_t)n / 8);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
// RMSNorm backward with library-owned scratch (see rmsnorm_bwd_static.h for the contract). Nothing above this
// line is changed by it; it goes through the same launcher as sb_rmsnorm_bwd with `dw_partial` pointing into the
// array below.
#include <atomic>
#include <cstdio>

#include "rmsnorm_bwd_static.h"

static_assert(SB_RMSNORM_STATIC_MAX_H == sb::NORM_THREADS * sb::NORM_MAX_VEC * 8,
              "the static scratch is sized for the widest row the norm kernels accept");

// [SB_RMSNORM_STATIC_MAX_CTAS, SB_RMSNORM_STATIC_MAX_H] fp32, 4.6 MiB. In host code this name is only a host-side
// stand-in for the symbol; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) float g_rmsnorm_bwd_static_scratch[SB_RMSNORM_STATIC_MAX_CTAS * SB_RMSNORM_STATIC_MAX_H];

namespace {
constexpr int kStaticMaxDevices = 64;
std::atomic<float*> g_static_scratch_addr[kStaticMaxDevices];  // zero-initialised; one slot per device ordinal

// Writes straight into the thread's message buffer: no std::string, no heap.
template <typename... A>
void static_fail(const char* fmt, A... a) {
  std::snprintf(sb::last_error_buf(), 512, fmt, a...);
}

// Returns the cached device address of the scratch for the current device, looking it up on first use.
int static_scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    static_fail("sb_rmsnorm_bwd_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
    return (int)e;
  }
  if (dev < 0 || dev >= kStaticMaxDevices) {
    static_fail("sb_rmsnorm_bwd_static: device ordinal %d is outside the supported range [0, %d)", dev, kStaticMaxDevices);
    return (int)cudaErrorInvalidDevice;
  }
  float* p = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    void* sym = nullptr;
    e = cudaGetSymbolAddress(&sym, g_rmsnorm_bwd_static_scratch);
    if (e != cudaSuccess || sym == nullptr) {
      static_fail("sb_rmsnorm_bwd_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : (int)cudaErrorInvalidSymbol;
    }
    p = static_cast<float*>(sym);
    g_static_scratch_addr[dev].store(p, std::memory_order_release);  // a concurrent first call stores the same value
  }
  *out = p;
  return 0;
}
}  // namespace

extern "C" int sb_rmsnorm_bwd_static_setup(void) {
  float* p = nullptr;
  return static_scratch_for_current_device(&p);
}

extern "C" int sb_rmsnorm_bwd_static(const void* dy, const void* h, const void* w, const float* rstd, const void* dres_in,
                                     void* dh, float* dw, int T, int H, int accumulate_dw, cudaStream_t s) {
  if (T < 0 || H <= 0 || H % 8 != 0 || H > SB_RMSNORM_STATIC_MAX_H) {
    static_fail("sb_rmsnorm_bwd_static: T=%d H=%d rejected; H must be a positive multiple of 8 and at most %d "
                "(scratch is %d x %d floats)", T, H, SB_RMSNORM_STATIC_MAX_H, SB_RMSNORM_STATIC_MAX_CTAS,
                SB_RMSNORM_STATIC_MAX_H);
    return (int)cudaErrorInvalidValue;
  }
  if (T == 0) return 0;
  if (dy == nullptr || h == nullptr || w == nullptr || rstd == nullptr || dh == nullptr || dw == nullptr) {
    static_fail("sb_rmsnorm_bwd_static: null pointer among dy/h/w/rstd/dh/dw");
    return (int)cudaErrorInvalidValue;
  }
  // The kernels move 16 bytes at a time through dy, h, w, dres_in and dh (rows are H * 2 bytes, a multiple of 16
  // because H % 8 == 0) and 4 bytes through rstd and dw: a base pointer off those boundaries would fault on the device,
  // so it is turned away here.
  auto misaligned = [](const void* p, uintptr_t a) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; };
  if (misaligned(dy, 16) || misaligned(h, 16) || misaligned(w, 16) || misaligned(dres_in, 16) || misaligned(dh, 16) ||
      misaligned(rstd, 4) || misaligned(dw, 4)) {
    static_fail("sb_rmsnorm_bwd_static: misaligned pointer; dy, h, w, dres_in and dh must be 16-byte aligned, rstd and dw "
                "4-byte aligned (H <= %d)", SB_RMSNORM_STATIC_MAX_H);
    return (int)cudaErrorInvalidValue;
  }
  float* scratch = nullptr;
  if (int rc = static_scratch_for_current_device(&scratch)) return rc;
  const int num_ctas = T < SB_RMSNORM_STATIC_MAX_CTAS ? T : SB_RMSNORM_STATIC_MAX_CTAS;
  // Rows of the scratch are packed with pitch H (not MAX_H), exactly like the caller-supplied buffer of sb_rmsnorm_bwd.
  cudaError_t e = sb::launch_rmsnorm_bwd((const bf16*)dy, (const bf16*)h, (const bf16*)w, rstd, (const bf16*)dres_in,
                                         (bf16*)dh, scratch, dw, T, H, num_ctas, accumulate_dw, s);
  if (e != cudaSuccess) static_fail("sb_rmsnorm_bwd_static: launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}
