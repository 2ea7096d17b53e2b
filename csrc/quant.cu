// Quantisation kernels (sm_100a).
//   * block-scaled e4m3 cast with BM x BN (default 128 x 128) fp32 scales, the weight-sync
//     quantiser: scale = max(absmax, 1e-10) / 448, q = clamp(x / scale); an all-zero block
//     yields q = 0 (no NaN). Optional power-of-two (UE8M0-representable) scales.
//   * e4m3 block dequant back to bf16
//   * fake INT4 quant-dequant for QAT with group shapes [1,g] / [g,1] / [bm,bn]
//   * small-M fp32-accumulate router GEMM (batch-invariant: fixed K order per output)
#include <cuda_fp8.h>

#include "common.cuh"

namespace sb {

// One CTA per (block_row, block_col); 256 threads sweep the BM x BN tile twice (absmax, cast).
__global__ void __launch_bounds__(256)
block_fp8_quant_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_e4m3* __restrict__ q, float* __restrict__ scale_inv,
                       int M, int N, size_t ldx, size_t ldq, int BM, int BN, int pow2_scale) {
  __shared__ float scratch[32];
  const int br = blockIdx.y, bc = blockIdx.x;
  const int r0 = br * BM, c0 = bc * BN;
  const int rows = min(BM, M - r0), cols = min(BN, N - c0);
  float amax = 0.f;
  for (int i = threadIdx.x; i < rows * cols; i += 256) {
    const int r = i / cols, c = i % cols;
    amax = fmaxf(amax, fabsf(__bfloat162float(x[(size_t)(r0 + r) * ldx + c0 + c])));
  }
  amax = block_max<256>(amax, scratch);
  float scale = fmaxf(amax, 1e-10f) / 448.f;
  if (pow2_scale) scale = exp2f(ceilf(log2f(scale)));
  if (threadIdx.x == 0) scale_inv[(size_t)br * gridDim.x + bc] = scale;  // "weight_scale_inv": multiply q by it
  const float inv = 1.f / scale;
  for (int i = threadIdx.x; i < rows * cols; i += 256) {
    const int r = i / cols, c = i % cols;
    float v = __bfloat162float(x[(size_t)(r0 + r) * ldx + c0 + c]) * inv;
    v = fminf(fmaxf(v, -448.f), 448.f);
    q[(size_t)(r0 + r) * ldq + c0 + c] = __nv_fp8_e4m3(v);
  }
}

// 1 x 128 groups (activation quantisation): one warp per group, lane = 4 consecutive elements. Scales go to
// scale_inv[row, group] and, when scale_t is given, also to scale_t[group, row] (the layout the fp8 GEMM reads).
__global__ void __launch_bounds__(256)
group_fp8_quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_e4m3* __restrict__ q, float* __restrict__ scale_inv,
                             float* __restrict__ scale_t, int M, int groups, size_t ldx, size_t ldq, int pow2_scale) {
  const int lane = threadIdx.x & 31;
  const size_t total = static_cast<size_t>(M) * groups;
  for (size_t g = static_cast<size_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); g < total; g += static_cast<size_t>(gridDim.x) * 8) {
    const size_t row = g / groups;
    const int grp = static_cast<int>(g - row * groups);
    const uint2 u = *reinterpret_cast<const uint2*>(x + row * ldx + grp * 128 + lane * 4);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
    amax = warp_max(amax);
    float scale = fmaxf(amax, 1e-10f) / 448.f;
    if (pow2_scale) scale = exp2f(ceilf(log2f(scale)));
    const float inv = 1.f / scale;
    if (lane == 0) {
      scale_inv[g] = scale;
      if (scale_t != nullptr) scale_t[static_cast<size_t>(grp) * M + row] = scale;
    }
    const float v[4] = {a.x * inv, a.y * inv, b.x * inv, b.y * inv};
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_fp8_e4m3 f(fminf(fmaxf(v[i], -448.f), 448.f));
      packed |= static_cast<uint32_t>(*reinterpret_cast<const uint8_t*>(&f)) << (8 * i);
    }
    *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(q) + row * ldq + grp * 128 + lane * 4) = packed;
  }
}

__global__ void __launch_bounds__(256)
block_fp8_dequant_kernel(const __nv_fp8_e4m3* __restrict__ q, const float* __restrict__ scale_inv,
                         __nv_bfloat16* __restrict__ out, int M, int N, int BM, int BN, int nbc) {
  const size_t n = (size_t)M * N;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / N), c = (int)(i % N);
    out[i] = __float2bfloat16(float(q[i]) * scale_inv[(size_t)(r / BM) * nbc + c / BN]);
  }
}

// Fake INT4: symmetric: s = absmax/7, y = clamp(rint(x/s), -8, 7)*s ; asymmetric: s = (max-min)/15,
// z = clamp(rint(-min/s), 0, 15), y = (clamp(rint(x/s)+z, 0, 15) - z)*s. One CTA per [gm x gn] group tile
// row-strip: grid.x = ceil(N/gn), grid.y = ceil(M/gm); group elements swept by the CTA.
__global__ void __launch_bounds__(128)
fake_int4_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, float* __restrict__ scales,
                 float* __restrict__ zeros, int M, int N, int gm, int gn, int symmetric) {
  __shared__ float scratch[32];
  const int r0 = blockIdx.y * gm, c0 = blockIdx.x * gn;
  const int rows = min(gm, M - r0), cols = min(gn, N - c0);
  float mx = -INFINITY, mn = INFINITY;
  for (int i = threadIdx.x; i < rows * cols; i += 128) {
    const float v = __bfloat162float(x[(size_t)(r0 + i / cols) * N + c0 + i % cols]);
    mx = fmaxf(mx, v);
    mn = fminf(mn, v);
  }
  mx = block_max<128>(mx, scratch);
  mn = -block_max<128>(-mn, scratch);
  float s, z = 0.f;
  if (symmetric) {
    s = fmaxf(fmaxf(fabsf(mx), fabsf(mn)), 1e-8f) / 7.f;
  } else {
    s = fmaxf(mx - mn, 1e-8f) / 15.f;
    z = fminf(fmaxf(rintf(-mn / s), 0.f), 15.f);
  }
  if (threadIdx.x == 0) {
    const size_t gi = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
    if (scales != nullptr) scales[gi] = s;
    if (zeros != nullptr) zeros[gi] = z;
  }
  for (int i = threadIdx.x; i < rows * cols; i += 128) {
    const size_t idx = (size_t)(r0 + i / cols) * N + c0 + i % cols;
    const float v = __bfloat162float(x[idx]);
    float qv;
    if (symmetric)
      qv = fminf(fmaxf(rintf(v / s), -8.f), 7.f) * s;
    else
      qv = (fminf(fmaxf(rintf(v / s) + z, 0.f), 15.f) - z) * s;
    y[idx] = __float2bfloat16(qv);
  }
}

// out[t, e] = sum_k in[t, k] * W[e, k]; bf16 inputs, fp32 output. grid = E experts, one CTA per
// expert row computes all M <= 16 tokens so every output has the same fixed reduction order
// regardless of batch composition (grid.y walks the tokens in chunks of 16).
constexpr int ROUTER_MAX_M = 16;
__global__ void __launch_bounds__(128)
router_gemm_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ W, float* __restrict__ out, int M,
                   int K, int E) {
  __shared__ float red[ROUTER_MAX_M][4];
  const int e = blockIdx.x;
  const int m_base = blockIdx.y * ROUTER_MAX_M;
  in += (size_t)m_base * K;
  out += (size_t)m_base * E;
  M = min(ROUTER_MAX_M, M - m_base);
  float acc[ROUTER_MAX_M];
#pragma unroll
  for (int m = 0; m < ROUTER_MAX_M; ++m) acc[m] = 0.f;
  const uint4* wrow = reinterpret_cast<const uint4*>(W + (size_t)e * K);
  for (int c = threadIdx.x; c < (K >> 3); c += 128) {
    const uint4 wu = wrow[c];
    const float2 w0 = unpack_bf16x2(wu.x), w1 = unpack_bf16x2(wu.y), w2 = unpack_bf16x2(wu.z), w3 = unpack_bf16x2(wu.w);
#pragma unroll
    for (int m = 0; m < ROUTER_MAX_M; ++m) {
      if (m < M) {
        const uint4 xu = reinterpret_cast<const uint4*>(in + (size_t)m * K)[c];
        const float2 x0 = unpack_bf16x2(xu.x), x1 = unpack_bf16x2(xu.y), x2 = unpack_bf16x2(xu.z), x3 = unpack_bf16x2(xu.w);
        acc[m] += x0.x * w0.x + x0.y * w0.y + x1.x * w1.x + x1.y * w1.y + x2.x * w2.x + x2.y * w2.y + x3.x * w3.x +
                  x3.y * w3.y;
      }
    }
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int m = 0; m < ROUTER_MAX_M; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0) red[m][wid] = v;
  }
  __syncthreads();
  if (threadIdx.x < M) {
    const int m = threadIdx.x;
    out[(size_t)m * E + e] = (red[m][0] + red[m][1]) + (red[m][2] + red[m][3]);
  }
}

}  // namespace sb

extern "C" int sb_block_fp8_quant(const void* x, void* q, float* scale_inv, int M, int N, long ldx, long ldq, int BM,
                                  int BN, int pow2_scale, cudaStream_t s) {
  if (M == 0 || N == 0) return 0;
  if (BM == 1 && BN == 128 && N % 128 == 0 && ldx % 4 == 0 && ldq % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 7) == 0 &&
      (reinterpret_cast<uintptr_t>(q) & 3) == 0) {
    const long total = (long)M * (N / 128);
    long blocks = (total + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    sb::group_fp8_quant_1x128_kernel<<<(int)blocks, 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_fp8_e4m3*)q, scale_inv, nullptr,
                                                                 M, N / 128, (size_t)ldx, (size_t)ldq, pow2_scale);
    return (int)cudaGetLastError();
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  sb::block_fp8_quant_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_fp8_e4m3*)q, scale_inv, M, N, (size_t)ldx,
                                                 (size_t)ldq, BM, BN, pow2_scale);
  return (int)cudaGetLastError();
}

// 1 x 128 activation quantisation that also writes the scales K-block major ([N/128, M]) for sb_gemm_fp8_block.
extern "C" int sb_group_fp8_quant_1x128(const void* x, void* q, float* scale_inv, float* scale_t, int M, int N, long ldx,
                                        long ldq, int pow2_scale, cudaStream_t s) {
  if (M == 0 || N == 0) return 0;
  if (N % 128 != 0 || ldx % 4 != 0 || ldq % 4 != 0 || (reinterpret_cast<uintptr_t>(x) & 7) != 0 ||
      (reinterpret_cast<uintptr_t>(q) & 3) != 0)
    return (int)cudaErrorInvalidValue;
  const long total = (long)M * (N / 128);
  long blocks = (total + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  sb::group_fp8_quant_1x128_kernel<<<(int)blocks, 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_fp8_e4m3*)q, scale_inv, scale_t, M,
                                                               N / 128, (size_t)ldx, (size_t)ldq, pow2_scale);
  return (int)cudaGetLastError();
}

extern "C" int sb_block_fp8_dequant(const void* q, const float* scale_inv, void* out, int M, int N, int BM, int BN,
                                    cudaStream_t s) {
  if (M == 0 || N == 0) return 0;
  sb::block_fp8_dequant_kernel<<<148 * 8, 256, 0, s>>>((const __nv_fp8_e4m3*)q, scale_inv, (__nv_bfloat16*)out, M, N, BM,
                                                      BN, (N + BN - 1) / BN);
  return (int)cudaGetLastError();
}

extern "C" int sb_fake_int4(const void* x, void* y, float* scales, float* zeros, int M, int N, int gm, int gn,
                            int symmetric, cudaStream_t s) {
  if (M == 0 || N == 0) return 0;
  dim3 grid((N + gn - 1) / gn, (M + gm - 1) / gm);
  sb::fake_int4_kernel<<<grid, 128, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, scales, zeros, M, N, gm, gn,
                                            symmetric);
  return (int)cudaGetLastError();
}

extern "C" int sb_router_gemm(const void* in, const void* W, float* out, int M, int K, int E, cudaStream_t s) {
  if (M == 0) return 0;
  if (K % 8 != 0) return (int)cudaErrorInvalidValue;
  dim3 grid(E, (M + sb::ROUTER_MAX_M - 1) / sb::ROUTER_MAX_M);
  sb::router_gemm_kernel<<<grid, 128, 0, s>>>((const __nv_bfloat16*)in, (const __nv_bfloat16*)W, out, M, K, E);
  return (int)cudaGetLastError();
}
