// Block-scaled FP8 (e4m3) GEMM for sm_100a: C[M, N] = (A ∘ sa) · (B ∘ sb)^T, bf16 or fp32 out.
//
//   A [M, K] e4m3 row-major, one fp32 scale per (row, 128-wide K block):      sa_t [K/128, M]   (K-block major)
//   B [N, K] e4m3 row-major, one fp32 scale per (128-row, 128-wide K) block:  sb   [ceil(N/128), K/128]
//   (the layout of a block-quantised checkpoint and of 1x128 activation quantisation)
//
// Because the scales change every 128 elements of K, each K block is multiplied on its own: four
// tcgen05.mma.kind::f8f6f4 (128x256x32) fill a fresh TMEM accumulator, and the epilogue warps fold it into fp32
// registers as acc += partial * sa[row] * sb[block] ("promotion") while the tensor core already works on the next K
// block in the other TMEM accumulator. Warp roles: 0 = TMA producer (4-stage ring of 16 KB A + 32 KB B tiles,
// 128-byte swizzle: one smem row = one K block), 1 = MMA issuer, 2..9 = promotion + store (two warps per TMEM lane
// quarter, one per 128-column half of the 128 x 256 tile, i.e. per B scale block; thread = output row, 128 fp32
// accumulators in registers). Persistent over output tiles. Grouped form (expert MLPs): B is a stack of E matrices
// [E * N, K] with scales [E, ceil(N/128), K/128]; every 128-row tile of A belongs to one expert and `tile_boff[m-tile]`
// is that expert's first row in the stack. Every wait is bounded: on expiry the CTA records a status word,
// stops issuing, frees its TMEM and returns.
#include <string>

#include "common.cuh"

namespace sb {

constexpr int F8_BM = 128, F8_BN = 256, F8_BK = 128;  // BK in elements = bytes; BN = two 128-wide scale blocks
constexpr int F8_STAGES = 4;
constexpr int F8_NACC = 2;     // TMEM accumulators in flight (2 x 256 columns = all of TMEM)
constexpr int F8_PANEL_M = 16;  // m-tiles per rasterisation panel
constexpr int F8_THREADS = 320;  // producer warp, MMA warp, 8 promotion warps
constexpr int F8_A_BYTES = F8_BM * F8_BK, F8_B_BYTES = F8_BN * F8_BK;  // 16 KB + 32 KB per stage
constexpr int F8_STAGE_BYTES = F8_A_BYTES + F8_B_BYTES;
constexpr int F8_SMEM = F8_STAGES * F8_STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;

// Tiles are walked panel by panel: 16 m-tiles wide, m fastest inside a panel, so the ~148 tiles in flight touch about
// 16 A row-blocks and 9 B row-blocks (25 x 128 x K bytes, L2-resident) instead of one B block and 148 A blocks.
__device__ __forceinline__ void f8_tile_origin(int tile, int tiles_m, int tiles_n, int& m0, int& n0) {
  const int per_panel = F8_PANEL_M * tiles_n;
  const int panel = tile / per_panel, r = tile - panel * per_panel;
  const int pm = min(F8_PANEL_M, tiles_m - panel * F8_PANEL_M);  // the last panel may be narrower
  m0 = (panel * F8_PANEL_M + r % pm) * F8_BM;
  n0 = (r / pm) * F8_BN;
}

template <bool OUT_F32>
__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const float* __restrict__ sa_t, const float* __restrict__ sb, void* __restrict__ Cv, int M, int N,
                      int K, int ldc, const int* __restrict__ tile_boff, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + F8_STAGES * F8_A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + F8_STAGES * F8_STAGE_BYTES);
  uint64_t* empty = full + F8_STAGES;
  uint64_t* acc_full = empty + F8_STAGES;
  uint64_t* acc_empty = acc_full + F8_NACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + F8_NACC);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + F8_BM - 1) / F8_BM, tiles_n = (N + F8_BN - 1) / F8_BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = K / F8_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < F8_NACC; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 8);  // one arrival per promotion warp
    }
    *cta_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, F8_NACC * F8_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m0, n0;
        f8_tile_origin(tile, tiles_m, tiles_n, m0, n0);
        const int boff = tile_boff != nullptr ? __ldg(tile_boff + m0 / F8_BM) : 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, cta_abort, status, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[stage], F8_STAGE_BYTES);
          tma_load_2d(sA + stage * F8_A_BYTES, &tmA, &full[stage], kb * F8_BK, m0);
          tma_load_2d(sB + stage * F8_B_BYTES, &tmB, &full[stage], kb * F8_BK, n0 + boff);
          if (++stage == F8_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(F8_BM, F8_BN, 0, 0, 0, 0);  // e4m3 x e4m3, both K-major
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, cta_abort, status, ERR_WAIT_TMEM_EMPTY) ||
              !mbar_wait(&full[stage], phase, cta_abort, status, ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * F8_A_BYTES), b_addr = smem_u32(sB + stage * F8_B_BYTES);
#pragma unroll
          for (int k = 0; k < F8_BK / 32; ++k)  // 32 fp8 elements = 32 bytes along the swizzled row per instruction
            umma_f8(tmem_base + acc * F8_BN, make_smem_desc(a_addr + k * 32, 16, 1024, UMMA_SWIZZLE_128B),
                    make_smem_desc(b_addr + k * 32, 16, 1024, UMMA_SWIZZLE_128B), idesc, k != 0 ? 1u : 0u);
          umma_commit(&empty[stage]);
          umma_commit(&acc_full[acc]);
          if (++stage == F8_STAGES) {
            stage = 0;
            phase ^= 1;
          }
          if (++acc == F8_NACC) {
            acc = 0;
            acc_phase ^= 1;
          }
        }
      }
    }
  } else {
    constexpr int HALF = F8_BN / 2;  // 128 columns = one scale block of B
    const int q = warp & 3;          // TMEM lane quarter of this warp
    const int h = (warp - 2) >> 2;   // which 128-column half of the tile
    const int row_in_tile = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m0, n0;
      f8_tile_origin(tile, tiles_m, tiles_n, m0, n0);
      const int row = m0 + row_in_tile;
      const int nblk = min(n0 / 128 + h, (N + 127) / 128 - 1);  // a tile's second half may lie past N: its scales are unused
      // grouped: the expert's own scale table ([ceil(N/128), K/128] per expert)
      const int expert = tile_boff != nullptr ? __ldg(tile_boff + m0 / F8_BM) / N : 0;
      const float* sb_row = sb + (static_cast<size_t>(expert) * ((N + 127) / 128) + nblk) * num_kb;
      float c[HALF];
#pragma unroll
      for (int i = 0; i < HALF; ++i) c[i] = 0.f;
      // the scales of a K block are fetched two blocks ahead: a global load issued inside the iteration that needs it
      // would put its full latency on the critical path of every block
      auto load_scale = [&](int kb) -> float {
        if (kb >= num_kb) return 0.f;
        return (row < M ? __ldg(sa_t + static_cast<size_t>(kb) * M + row) : 0.f) * __ldg(sb_row + kb);
      };
      float s_cur = load_scale(0), s_next = load_scale(1);
      for (int kb = 0; kb < num_kb; ++kb) {
        const float s = s_cur;
        s_cur = s_next;
        s_next = load_scale(kb + 2);
        ok = mbar_wait(&acc_full[acc], acc_phase, cta_abort, status, ERR_WAIT_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t t = tmem_base + acc * F8_BN + h * HALF + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t + pass * 64, r0);  // both loads in flight before the wait
          tmem_ld_32x32(t + pass * 64 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            c[pass * 64 + i] = fmaf(__uint_as_float(r0[i]), s, c[pass * 64 + i]);
            c[pass * 64 + 32 + i] = fmaf(__uint_as_float(r1[i]), s, c[pass * 64 + 32 + i]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        if (++acc == F8_NACC) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
      const int col0 = n0 + h * HALF;
      if (ok && row < M && col0 < N) {
        if constexpr (OUT_F32) {
          float* dst = static_cast<float*>(Cv) + static_cast<size_t>(row) * ldc + col0;
          if (col0 + HALF <= N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < HALF; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(c[i], c[i + 1], c[i + 2], c[i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < HALF; ++i)
              if (col0 + i < N) dst[i] = c[i];
          }
        } else {
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(Cv) + static_cast<size_t>(row) * ldc + col0;
          if (col0 + HALF <= N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < HALF; i += 8) {
              uint4 o;
              o.x = pack_bf16x2(c[i], c[i + 1]); o.y = pack_bf16x2(c[i + 2], c[i + 3]);
              o.z = pack_bf16x2(c[i + 4], c[i + 5]); o.w = pack_bf16x2(c[i + 6], c[i + 7]);
              *reinterpret_cast<uint4*>(dst + i) = o;
            }
          } else {
#pragma unroll
            for (int i = 0; i < HALF; ++i)
              if (col0 + i < N) dst[i] = __float2bfloat16(c[i]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, F8_NACC * F8_BN);
}

}  // namespace sb

// A, B: e4m3 bytes, row-major with pitches lda / ldb (bytes = elements; multiples of 16). sa_t: [K/128, M] fp32.
// sb: [ceil(N/128), K/128] fp32. C: [M, N] bf16 (out_f32 = 0) or fp32, pitch ldc elements. K must be a multiple of 128.
// Grouped (tile_boff != nullptr): B is [num_experts * N, K], sb is [num_experts, ceil(N/128), K/128], M a multiple of 128
// and tile_boff[M / 128] the first stack row of each row tile's expert.
static int fp8_launch(const void* A, const void* B, const float* sa_t, const float* sb, void* C, int M, int N, int K, int lda,
                      int ldb, int ldc, int out_f32, const int* tile_boff, int num_experts, int* status, int num_sms,
                      cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % sb::F8_BK != 0 || lda % 16 != 0 || ldb % 16 != 0) {
    sb::set_last_error("sb_gemm_fp8_block: K must be a multiple of 128 and the row pitches multiples of 16 bytes");
    return (int)cudaErrorInvalidValue;
  }
  if (tile_boff != nullptr && (M % sb::F8_BM != 0 || num_experts <= 0)) {
    sb::set_last_error("sb_gemm_fp8_grouped: M must be a multiple of 128 (expert-padded rows) and num_experts positive");
    return (int)cudaErrorInvalidValue;
  }
  try {
    CUtensorMap tmA = sb::make_tmap_2d(A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, size_t(lda), sb::F8_BM, sb::F8_BK,
                                       CU_TENSOR_MAP_SWIZZLE_128B);
    const size_t b_rows = tile_boff != nullptr ? size_t(num_experts) * N : size_t(N);
    CUtensorMap tmB = sb::make_tmap_2d(B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_rows, K, size_t(ldb), sb::F8_BN, sb::F8_BK,
                                       CU_TENSOR_MAP_SWIZZLE_128B);
    const int tiles = ((M + sb::F8_BM - 1) / sb::F8_BM) * ((N + sb::F8_BN - 1) / sb::F8_BN);
    const int grid = tiles < num_sms ? tiles : num_sms;
    cudaError_t e;
    if (out_f32) {
      e = sb::ensure_dynamic_smem(reinterpret_cast<const void*>(sb::gemm_fp8_block_kernel<true>), sb::F8_SMEM);
      if (e != cudaSuccess) return (int)e;
      e = sb::launch_pdl(sb::gemm_fp8_block_kernel<true>, dim3(grid), dim3(sb::F8_THREADS), sb::F8_SMEM, stream, tmA, tmB, sa_t,
                         sb, C, M, N, K, ldc, tile_boff, status);
    } else {
      e = sb::ensure_dynamic_smem(reinterpret_cast<const void*>(sb::gemm_fp8_block_kernel<false>), sb::F8_SMEM);
      if (e != cudaSuccess) return (int)e;
      e = sb::launch_pdl(sb::gemm_fp8_block_kernel<false>, dim3(grid), dim3(sb::F8_THREADS), sb::F8_SMEM, stream, tmA, tmB,
                         sa_t, sb, C, M, N, K, ldc, tile_boff, status);
    }
    if (e != cudaSuccess) sb::set_last_error(std::string("fp8 gemm launch: ") + cudaGetErrorString(e));
    return (int)e;
  } catch (const std::exception& e) {
    sb::set_last_error(e.what());
    return (int)cudaErrorInvalidValue;
  }
}

extern "C" int sb_gemm_fp8_block(const void* A, const void* B, const float* sa_t, const float* sb, void* C, int M, int N,
                                 int K, int lda, int ldb, int ldc, int out_f32, int* status, int num_sms,
                                 cudaStream_t stream) {
  return fp8_launch(A, B, sa_t, sb, C, M, N, K, lda, ldb, ldc, out_f32, nullptr, 0, status, num_sms, stream);
}

extern "C" int sb_gemm_fp8_grouped(const void* A, const void* B, const float* sa_t, const float* sb, void* C,
                                   const int* tile_boff, int M, int N, int K, int num_experts, int lda, int ldb, int ldc,
                                   int out_f32, int* status, int num_sms, cudaStream_t stream) {
  if (tile_boff == nullptr) {
    sb::set_last_error("sb_gemm_fp8_grouped: needs tile_boff");
    return (int)cudaErrorInvalidValue;
  }
  return fp8_launch(A, B, sa_t, sb, C, M, N, K, lda, ldb, ldc, out_f32, tile_boff, num_experts, status, num_sms, stream);
}
