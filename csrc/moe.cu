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
