// Token <-> route permutation for mixture-of-experts layers, deterministic by construction: no atomics, every output
// element has exactly one writer, and sums over a token's k routes run in route order.
//
//   sb_moe_scatter_rows   out[dest[s], :] = x[s / k, :]                for every route slot s with dest[s] >= 0
//                         (tokens copied into the expert-sorted, tile-padded buffer the grouped GEMM reads)
//   sb_moe_gather_sum     y[t, :] = sum_{j<k} w[t*k+j] * rows[dest[t*k+j], :]   (routes with dest < 0 are skipped)
//                         fp32 accumulation in route order j = 0..k-1; with round_each the running sum is rounded to
//                         bf16 after every route, which reproduces a chain of bf16 adds bit for bit.
//                         This is the combine step of the forward pass and, with w = null, the gradient of the scatter.
//   sb_moe_route_weight_grad   dw[s] = <rows[dest[s], :], dy[s / k, :]>    (gradient of the combine w.r.t. the weights)
//
// One warp per slot (scatter, weight grad) or per token (gather); lanes stride over the row in 16-byte vectors.
#include "common.cuh"

namespace sb {

__global__ void __launch_bounds__(256)
moe_scatter_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ dest, __nv_bfloat16* __restrict__ out,
                        long slots, int k, int H) {
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (long s = static_cast<long>(blockIdx.x) * 8 + (threadIdx.x >> 5); s < slots; s += static_cast<long>(gridDim.x) * 8) {
    const int d = dest[s];
    if (d < 0) continue;
    const uint4* src = reinterpret_cast<const uint4*>(x + (s / k) * H);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long>(d) * H);
    for (int c = lane; c < nvec; c += 32) dst[c] = src[c];
  }
}

__global__ void __launch_bounds__(256)
moe_gather_sum_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ dest, const float* __restrict__ w,
                      __nv_bfloat16* __restrict__ y, long T, int k, int H, int round_each) {
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (long t = static_cast<long>(blockIdx.x) * 8 + (threadIdx.x >> 5); t < T; t += static_cast<long>(gridDim.x) * 8) {
    for (int c = lane; c < nvec; c += 32) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int j = 0; j < k; ++j) {
        const int d = dest[t * k + j];
        if (d < 0) continue;
        const float wj = w != nullptr ? w[t * k + j] : 1.f;
        const uint4 u = reinterpret_cast<const uint4*>(rows + static_cast<long>(d) * H)[c];
        const float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
        const float v[8] = {a0.x, a0.y, a1.x, a1.y, a2.x, a2.y, a3.x, a3.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          acc[i] = fmaf(wj, v[i], acc[i]);
          if (round_each) acc[i] = __bfloat162float(__float2bfloat16(acc[i]));
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(y + t * H)[c] = o;
    }
  }
}

__global__ void __launch_bounds__(256)
moe_route_weight_grad_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ dest,
                             const __nv_bfloat16* __restrict__ dy, float* __restrict__ dw, long slots, int k, int H) {
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (long s = static_cast<long>(blockIdx.x) * 8 + (threadIdx.x >> 5); s < slots; s += static_cast<long>(gridDim.x) * 8) {
    const int d = dest[s];
    float acc = 0.f;
    if (d >= 0) {
      const uint4* a = reinterpret_cast<const uint4*>(rows + static_cast<long>(d) * H);
      const uint4* b = reinterpret_cast<const uint4*>(dy + (s / k) * H);
      for (int c = lane; c < nvec; c += 32) {
        const uint4 ua = a[c], ub = b[c];
        const float2 a0 = unpack_bf16x2(ua.x), a1 = unpack_bf16x2(ua.y), a2 = unpack_bf16x2(ua.z), a3 = unpack_bf16x2(ua.w);
        const float2 b0 = unpack_bf16x2(ub.x), b1 = unpack_bf16x2(ub.y), b2 = unpack_bf16x2(ub.z), b3 = unpack_bf16x2(ub.w);
        acc += a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
      }
    }
    acc = warp_sum(acc);  // fixed butterfly order: the same bits on every run
    if (lane == 0) dw[s] = acc;
  }
}

// Top-k routing in one pass over the router logits: one warp per token, each lane keeps E / 32 logits in registers.
//   mode 0  pick the k largest logits; weights = softmax over the picked logits (== renormalised top-k of the softmax)
//   mode 1  weights = softmax over all experts, pick the k largest, no renormalisation
//   mode 2  scores = sigmoid(logit); pick by score + bias (bias only steers the choice); weights = picked scores,
//           divided by their sum when `renorm`
// then weights *= scale. Ties go to the lower expert index. E <= 512.
constexpr int TOPK_MAX_PER_LANE = 16;
__global__ void __launch_bounds__(256)
moe_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ idx, float* __restrict__ wts,
                long T, int E, int k, int mode, int renorm, float scale) {
  const int lane = threadIdx.x & 31;
  for (long t = static_cast<long>(blockIdx.x) * 8 + (threadIdx.x >> 5); t < T; t += static_cast<long>(gridDim.x) * 8) {
    float raw[TOPK_MAX_PER_LANE], sel[TOPK_MAX_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < TOPK_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      raw[i] = e < E ? logits[t * E + e] : -INFINITY;
      mx = fmaxf(mx, raw[i]);
    }
    mx = warp_max(mx);
    float denom = 0.f;
    if (mode == 1) {
#pragma unroll
      for (int i = 0; i < TOPK_MAX_PER_LANE; ++i) denom += lane + 32 * i < E ? __expf(raw[i] - mx) : 0.f;
      denom = warp_sum(denom);
    }
#pragma unroll
    for (int i = 0; i < TOPK_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e >= E) {
        sel[i] = -INFINITY;
      } else if (mode == 2) {
        raw[i] = 1.f / (1.f + __expf(-raw[i]));  // from here on "raw" is the score that becomes the weight
        sel[i] = raw[i] + (bias != nullptr ? bias[e] : 0.f);
      } else {
        sel[i] = raw[i];
      }
    }
    float picked_w = 0.f;  // lane j < k ends up holding the weight of the j-th pick
    int picked_e = 0;
    float wsum = 0.f;
    for (int r = 0; r < k; ++r) {
      float bv = -INFINITY;
      int be = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < TOPK_MAX_PER_LANE; ++i)
        if (sel[i] > bv) {  // strict: the lowest index wins inside a lane (indices grow with i)
          bv = sel[i];
          be = lane + 32 * i;
        }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ov > bv || (ov == bv && oe < be)) {
          bv = ov;
          be = oe;
        }
      }
      // the owner of the winner publishes the value the weight is made of and retires the element
      float val = 0.f;
      if ((be & 31) == lane) {
#pragma unroll
        for (int i = 0; i < TOPK_MAX_PER_LANE; ++i)
          if (lane + 32 * i == be) {
            val = raw[i];
            sel[i] = -INFINITY;
          }
      }
      val = __shfl_sync(0xffffffffu, val, be & 31);
      float wv;
      if (mode == 0) wv = __expf(val - mx);          // normalised below by the sum over the picks
      else if (mode == 1) wv = __expf(val - mx) / denom;
      else wv = val;
      wsum += wv;
      if (lane == r) {
        picked_w = wv;
        picked_e = be;
      }
    }
    if (mode == 0) picked_w /= wsum;
    else if (mode == 2 && renorm) picked_w /= (wsum + 1e-20f);
    if (lane < k) {
      idx[t * k + lane] = picked_e;
      wts[t * k + lane] = picked_w * scale;
    }
  }
}

static inline int moe_blocks(long items) {
  long b = (items + 7) / 8;
  return static_cast<int>(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace sb

// All row widths H must be multiples of 8 (16-byte vectors); pointers 16-byte aligned; rows contiguous (pitch H).
extern "C" int sb_moe_scatter_rows(const void* x, const int* dest, void* out, long slots, int k, int H, cudaStream_t s) {
  if (slots == 0) return 0;
  if (H % 8 != 0 || k <= 0) return (int)cudaErrorInvalidValue;
  sb::moe_scatter_rows_kernel<<<sb::moe_blocks(slots), 256, 0, s>>>((const __nv_bfloat16*)x, dest, (__nv_bfloat16*)out, slots, k, H);
  return (int)cudaGetLastError();
}

extern "C" int sb_moe_gather_sum(const void* rows, const int* dest, const float* w, void* y, long T, int k, int H,
                                 int round_each, cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8 != 0 || k <= 0) return (int)cudaErrorInvalidValue;
  sb::moe_gather_sum_kernel<<<sb::moe_blocks(T), 256, 0, s>>>((const __nv_bfloat16*)rows, dest, w, (__nv_bfloat16*)y, T, k, H,
                                                             round_each);
  return (int)cudaGetLastError();
}

extern "C" int sb_moe_route_weight_grad(const void* rows, const int* dest, const void* dy, float* dw, long slots, int k, int H,
                                        cudaStream_t s) {
  if (slots == 0) return 0;
  if (H % 8 != 0 || k <= 0) return (int)cudaErrorInvalidValue;
  sb::moe_route_weight_grad_kernel<<<sb::moe_blocks(slots), 256, 0, s>>>((const __nv_bfloat16*)rows, dest,
                                                                        (const __nv_bfloat16*)dy, dw, slots, k, H);
  return (int)cudaGetLastError();
}

// logits [T, E] fp32 (row-major, contiguous); bias [E] fp32 or null; idx [T, k] int32; weights [T, k] fp32. k <= 32.
extern "C" int sb_moe_topk(const float* logits, const float* bias, int* idx, float* weights, long T, int E, int k, int mode,
                           int renorm, float scale, cudaStream_t s) {
  if (T == 0) return 0;
  if (E <= 0 || E > 32 * sb::TOPK_MAX_PER_LANE || k <= 0 || k > 32 || k > E || mode < 0 || mode > 2)
    return (int)cudaErrorInvalidValue;
  sb::moe_topk_kernel<<<sb::moe_blocks(T), 256, 0, s>>>(logits, bias, idx, weights, T, E, k, mode, renorm, scale);
  return (int)cudaGetLastError();
}
