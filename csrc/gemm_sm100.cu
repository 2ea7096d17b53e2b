// bf16 GEMM for sm_100a: TMA-fed, tcgen05.mma with TMEM accumulators, persistent
// and warp-specialised.
//
//   C[M,N] (+)= op(A) * op(B)  (+ bias[N]),   fp32 accumulate, bf16 or fp32 output.
//
// op(A) is an M x K matrix given either K-major (row-major [M,K], the activation
// layout) or MN-major (stored [K,M], i.e. the transpose of a row-major tensor);
// likewise op(B) is N x K given K-major (row-major [N,K], the nn.Linear weight
// layout) or MN-major (stored [K,N]). This covers forward (X W^T), dgrad (dY W)
// and wgrad (dY^T X) without materialising any transpose.
//
// CTA = 6 warps: warp 0 issues TMA loads (one lane), warp 1 owns TMEM and issues
// tcgen05.mma (one lane), warps 2-5 drain the accumulators: tcgen05.ld -> registers ->
// (bias, cast) -> 128B-swizzled shared staging -> TMA store (or TMA reduce-add when
// accumulating into an fp32 C, e.g. wgrad into the main-grad buffer). Tile 128 x BN x 64,
// STAGES-deep smem ring, two TMEM accumulator stages so the epilogue of tile i overlaps
// the main loop of tile i+1. Grid = min(#tiles, #SMs).
// When C's pitch or base is not 16-byte aligned the epilogue falls back to direct,
// bounds-checked global stores.
#include "common.cuh"

namespace sb {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int GEMM_THREADS = 192;
constexpr int EPI_BUF_BYTES = 32 * 128;  // 32 rows x 128 B per staging buffer
constexpr int EPI_BYTES = 4 * 2 * EPI_BUF_BYTES;  // 4 epilogue warps x 2 buffers

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES + 1024;  // +1024: manual alignment
};

// Tile order. Tiles are walked in panels of GEMM_PANEL_M row-tiles: within a panel the m index runs fastest, then n.
// The ~148 tiles in flight at any time then share one A panel (kept in L2 while n sweeps) and a few B column
// blocks, so A is read from HBM once and B once per panel instead of both being re-fetched every wave.
constexpr int GEMM_PANEL_M = 32;

template <int BN>
__device__ __forceinline__ void tile_origin(int tile, int tiles_m, int tiles_n, int& m0, int& n0) {
  const int per_panel = GEMM_PANEL_M * tiles_n;
  const int panel = tile / per_panel;
  const int pm0 = panel * GEMM_PANEL_M;
  const int pm = min(GEMM_PANEL_M, tiles_m - pm0);
  const int r = tile - panel * per_panel;
  m0 = (pm0 + r % pm) * GEMM_BM;
  n0 = (r / pm) * BN;
}

// Optional extra kernel parameter: a collective fused into the GEMM over NVLink peer memory (no multicast loads).
//
// GatherA (all-gather -> GEMM, sequence-parallel column linear): the rows of A are spread over up to 8 GPUs, rank r
// holding rows [r * rows_per_rank, (r + 1) * rows_per_rank) in a buffer every rank can read. Four extra warps in every CTA
// pull the peers' shards ONCE into this GPU's `gathered` buffer (plain 16-byte loads from peer memory, 4-row pieces
// striped over the CTAs, nearest peer first) and counts the pieces of each 128-row block; the tile order starts with the
// rank's own rows, and the TMA producer waits (bounded) for a remote block's counter before it loads tiles of that
// block from LOCAL memory. Every remote byte crosses NVLink once, under the GEMM of the rows that are already there,
// and the gathered activation is left behind for the weight-gradient GEMM of the backward pass.
//
// ScatterC (GEMM -> reduce-scatter, sequence-parallel row linear): every rank computes the full [M, N] partial product;
// rows [o * rows_per_rank, ...) belong to rank o. The epilogue TMA-stores each bf16 tile into slot `rank` of the
// owner's receive buffer (its own or a peer's) and then raises one flag word per (tile, source rank, epilogue warp) on
// the owner; tiles owned by peers are computed first. When a CTA has finished its share of the GEMM its epilogue warps
// turn to the tiles this rank owns: wait (bounded) for every source's flag, sum the `world` slots in rank order in fp32
// and write the reduced bf16 tile. No NCCL call, no second launch, fixed summation order.
struct NoExtra {
  static constexpr int kMode = 0;
};
struct GatherA {
  static constexpr int kMode = 1;
  const void* peer[8];  // shard of rank r: [rows_per_rank, K] bf16, contiguous rows
  void* gathered;       // this GPU's [world * rows_per_rank, K] bf16, contiguous: the A operand (own rows filled by the caller)
  uint32_t* counters;   // one per 128-row block of `gathered`: pieces copied so far, monotonic over calls
  uint32_t target;      // value a block's counter has when this call's copy of the block is complete
  int rows_per_rank, world, rank, row_bytes;
  unsigned long long limit_ns;
};
struct ScatterC {
  static constexpr int kMode = 2;
  CUtensorMap slot[8];        // owner o's receive buffer viewed as [world * rows_per_rank, N] bf16 (slot-major)
  const __nv_bfloat16* recv;  // this rank's own receive buffer, same view
  uint32_t* flags[8];         // owner o's flag words: [owned tiles][world][4 epilogue warps]
  __nv_bfloat16* out;         // [rows_per_rank, N] bf16, pitch ld_out
  int ld_out;
  uint32_t epoch;
  int rows_per_rank, world, rank;
  unsigned long long limit_ns;
};
constexpr int GATHER_PIECE_ROWS = 4;
constexpr int GATHER_WARPS = 4;  // per CTA: enough 16-byte loads in flight over NVLink to run at link rate

__device__ __forceinline__ void st_release_sys_u32(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
// All of this thread's bulk groups have completed (their writes performed), not merely read their source.
__device__ __forceinline__ void bulk_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Order of the row tiles. rot > 0: the walk starts at tile `rot` and wraps (gathering: own rows first, while the
// peers' rows arrive). rot < 0, -rot = world << 8 | rank (scattering): consecutive positions of the walk belong to
// different owners (rank + 1, rank + 2, ..., rank), so the stores to the peers are spread over the whole GEMM instead of
// saturating NVLink during its first part, and every owner starts receiving at once.
template <int BN>
__device__ __forceinline__ void tile_origin_rot(int tile, int tiles_m, int tiles_n, int rot, int& m0, int& n0) {
  tile_origin<BN>(tile, tiles_m, tiles_n, m0, n0);
  if (rot > 0) {
    int mt = m0 / GEMM_BM + rot;
    if (mt >= tiles_m) mt -= tiles_m;
    m0 = mt * GEMM_BM;
  } else if (rot < 0) {
    const int world = (-rot) >> 8, rank = (-rot) & 0xff;
    const int mt = m0 / GEMM_BM, tpr = tiles_m / world;
    int owner = rank + 1 + mt % world;
    if (owner >= world) owner -= world;
    m0 = (owner * tpr + mt / world) * GEMM_BM;
  }
}

template <int BN, int STAGES, bool A_MN, bool B_MN, bool OUT_F32, bool TMA_EPI, typename Extra = NoExtra>
__global__ void __launch_bounds__(GEMM_THREADS + 32 * GATHER_WARPS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, void* __restrict__ Cv, const __nv_bfloat16* __restrict__ bias,
                 int M, int N, int K, int ldc, int accumulate, int* status, const int* __restrict__ tile_boff,
                 const __grid_constant__ Extra extra) {
  using S = GemmSmem<BN, STAGES>;
  constexpr int NCOLS = 2 * BN;  // two accumulator stages (power of two: 256 or 512)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * S::A_BYTES;
  uint8_t* sC = smem + STAGES * S::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(sC + EPI_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + GEMM_BK - 1) / GEMM_BK;
  // Split-K: `accumulate` carries the number of K slices in bits 8.. (1 = no split). A work item is (tile, slice); the
  // slices of a tile are summed by the epilogue's TMA reduce-add, so the caller passes a zeroed C or asks to accumulate.
  const int splitk = (accumulate >> 8) > 1 ? (accumulate >> 8) : 1;
  const bool add_out = (accumulate & 1) != 0 || splitk > 1;
  const int kb_per = (num_kb + splitk - 1) / splitk;
  const int num_items = num_tiles * splitk;
  int rot = 0;  // first row tile of the walk
  if constexpr (Extra::kMode == 1) rot = extra.rank * (extra.rows_per_rank / GEMM_BM);
  if constexpr (Extra::kMode == 2) rot = -((extra.world << 8) | extra.rank);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull[s], 1);
      mbar_init(&tempty[s], 4);  // one arrival per epilogue warp
    }
    *cta_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if constexpr (TMA_EPI) tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, NCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above (barriers, TMEM, descriptor prefetch) may overlap the previous kernel; operands may not.
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int tile = item / splitk, ks = item - tile * splitk;
        int m0, n0;
        tile_origin_rot<BN>(tile, tiles_m, tiles_n, rot, m0, n0);
        if constexpr (Extra::kMode == 1) {
          // rows of another rank: wait until the gather warps have brought the whole 128-row block into local memory
          if (m0 / extra.rows_per_rank != extra.rank) {
            const uint32_t* ctr = extra.counters + m0 / GEMM_BM;
            const unsigned long long t0 = globaltimer_ns();
            uint32_t it = 0;
            while (static_cast<int32_t>(ld_acquire_gpu_u32(ctr) - extra.target) < 0) {
              if ((++it & 0x3f) == 0) {
                if (*cta_abort) {
                  ok = false;
                  break;
                }
                if (globaltimer_ns() - t0 > extra.limit_ns) {
                  *cta_abort = 1;
                  if (status) atomicCAS(status, 0, ERR_WAIT_PEER | (blockIdx.x << 8));
                  ok = false;
                  break;
                }
              }
            }
            if (!ok) break;
            fence_proxy_async_all();  // rows written with plain stores by other CTAs -> visible to this TMA load
          }
        }
        // Grouped GEMM: B is the experts' matrices stacked along its row dimension and every 128-row tile of A belongs
        // to one expert; tile_boff[m-tile] is the row at which that expert's matrix starts in the stack.
        const int boff = tile_boff != nullptr ? __ldg(tile_boff + m0 / GEMM_BM) : 0;
        const int kb_end = min(num_kb, (ks + 1) * kb_per);
        for (int kb = ks * kb_per; kb < kb_end; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, cta_abort, status, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[stage], S::STAGE_BYTES);
          uint8_t* a_dst = sA + stage * S::A_BYTES;
          uint8_t* b_dst = sB + stage * S::B_BYTES;
          if constexpr (!A_MN) {
            tma_load_2d(a_dst, &tmA, &full[stage], kb * GEMM_BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j)
              tma_load_2d(a_dst + j * 8192, &tmA, &full[stage], m0 + j * 64, kb * GEMM_BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d(b_dst, &tmB, &full[stage], kb * GEMM_BK, n0 + boff);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * 8192, &tmB, &full[stage], n0 + j * 64, kb * GEMM_BK + boff);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(GEMM_BM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, cta_abort, status, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int ks = item % splitk;
        const int kb0 = ks * kb_per, kb_end = min(num_kb, (ks + 1) * kb_per);
        for (int kb = kb0; kb < kb_end; ++kb) {
          if (!mbar_wait(&full[stage], phase, cta_abort, status, ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * S::A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * S::B_BYTES);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            // K-major, 128B swizzle: 8-row groups 1024 B apart; a K step of 16 elements is 32 B inside the row.
            // MN-major, 128B swizzle: 64-element column chunks 8192 B apart (LBO), 8 k-rows = 1024 B (SBO);
            // a K step of 16 rows is 2048 B.
            const uint64_t da = A_MN ? make_smem_desc(a_addr + k * 2048, 8192, 1024, UMMA_SWIZZLE_128B)
                                     : make_smem_desc(a_addr + k * 32, 16, 1024, UMMA_SWIZZLE_128B);
            const uint64_t db = B_MN ? make_smem_desc(b_addr + k * 2048, 8192, 1024, UMMA_SWIZZLE_128B)
                                     : make_smem_desc(b_addr + k * 32, 16, 1024, UMMA_SWIZZLE_128B);
            umma_f16(d_tmem, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);  // frees the smem slot once these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tfull[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    uint8_t* stage_buf = sC + q * 2 * EPI_BUF_BYTES;
    int buf = 0;
    const __nv_bfloat16* const bias_all = bias;
    for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
      const int tile = item / splitk;
      const __nv_bfloat16* bias = (item - tile * splitk) == 0 ? bias_all : nullptr;  // one slice adds the bias
      int m0, n0;
      tile_origin_rot<BN>(tile, tiles_m, tiles_n, rot, m0, n0);
      bool ok = mbar_wait(&tfull[acc], acc_phase, cta_abort, status, ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      if constexpr (TMA_EPI) {
        // one box = 32 rows x 128 bytes: 64 bf16 columns or 32 fp32 columns
        constexpr int BOX_COLS = OUT_F32 ? 32 : 64;
        const int row0 = m0 + q * 32;
#pragma unroll 1
        for (int c = 0; c < BN / BOX_COLS; ++c) {
          const int col0 = n0 + c * BOX_COLS;
          // Boxes that lie wholly outside C are skipped as a whole (warp-uniform): every iteration that touches a
          // staging buffer also commits exactly one bulk group, which is what makes wait_group<1> mean "the store
          // that last read THIS buffer is done".
          if (row0 >= M || col0 >= N) break;
          uint8_t* dst = stage_buf + buf * EPI_BUF_BYTES;
          if (lane == 0) bulk_wait_group_read<1>();  // the store that last used this buffer has drained it
          __syncwarp();
          uint8_t* my_row = dst + lane * 128;
          const int sw = lane & 7;  // 128B swizzle: 16-byte chunk j of row r lives at chunk j ^ (r % 8)
          if constexpr (OUT_F32) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 o = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                     __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
              if (bias != nullptr) {
                const int cc = col0 + 4 * j;
                if (cc + 0 < N) o.x += __bfloat162float(bias[cc + 0]);
                if (cc + 1 < N) o.y += __bfloat162float(bias[cc + 1]);
                if (cc + 2 < N) o.z += __bfloat162float(bias[cc + 2]);
                if (cc + 3 < N) o.w += __bfloat162float(bias[cc + 3]);
              }
              *reinterpret_cast<float4*>(my_row + ((j ^ sw) << 4)) = o;
            }
          } else {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t r[32];
              tmem_ld_32x32(t_row + c * 64 + half * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[8 * j + i]);
                if (bias != nullptr) {
                  const int cc = col0 + half * 32 + 8 * j;
#pragma unroll
                  for (int i = 0; i < 8; ++i)
                    if (cc + i < N) v[i] += __bfloat162float(bias[cc + i]);
                }
                uint4 o;
                o.x = pack_bf16x2(v[0], v[1]);
                o.y = pack_bf16x2(v[2], v[3]);
                o.z = pack_bf16x2(v[4], v[5]);
                o.w = pack_bf16x2(v[6], v[7]);
                *reinterpret_cast<uint4*>(my_row + (((half * 4 + j) ^ sw) << 4)) = o;
              }
            }
          }
          fence_proxy_async();  // generic-proxy writes -> visible to the TMA engine
          __syncwarp();
          if (lane == 0) {
            if constexpr (Extra::kMode == 2) {
              const int owner = m0 / extra.rows_per_rank;
              tma_store_2d(&extra.slot[owner], dst, col0, row0 - owner * extra.rows_per_rank + extra.rank * extra.rows_per_rank);
            } else if (add_out) {
              tma_reduce_add_2d(&tmC, dst, col0, row0);
            } else {
              tma_store_2d(&tmC, dst, col0, row0);
            }
            bulk_commit_group();
          }
          buf ^= 1;
        }
        if constexpr (Extra::kMode == 2) {
          // the accumulator has been drained into the staging buffers: hand it back before waiting for the stores
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[acc]);
          // this warp's 32 rows of the tile are on their way: once the stores have completed, tell the owner
          if (lane == 0) {
            bulk_wait_group_all();
            fence_proxy_async_all();
            __threadfence_system();
            const int owner = m0 / extra.rows_per_rank;
            const int lt = ((m0 - owner * extra.rows_per_rank) / GEMM_BM) * tiles_n + n0 / BN;
            st_release_sys_u32(extra.flags[owner] + (static_cast<size_t>(lt) * extra.world + extra.rank) * 4 + q, extra.epoch);
          }
          __syncwarp();
        }
      } else {
        const int row = m0 + q * 32 + lane;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (row < M && col0 < N) {
            if constexpr (OUT_F32) {
              float* crow = reinterpret_cast<float*>(Cv) + static_cast<size_t>(row) * ldc + col0;
              for (int i = 0; i < 32 && col0 + i < N; ++i) {
                float v = __uint_as_float(r[i]);
                if (bias != nullptr) v += __bfloat162float(bias[col0 + i]);
                crow[i] = add_out ? crow[i] + v : v;
              }
            } else {
              __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cv) + static_cast<size_t>(row) * ldc + col0;
              for (int i = 0; i < 32 && col0 + i < N; ++i) {
                float v = __uint_as_float(r[i]);
                if (bias != nullptr) v += __bfloat162float(bias[col0 + i]);
                crow[i] = __float2bfloat16(v);
              }
            }
          }
        }
      }
      if constexpr (Extra::kMode != 2) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if constexpr (TMA_EPI) {
      if (lane == 0) bulk_wait_group_read<0>();  // staging memory must outlive the stores that read it
      __syncwarp();
    }
    if constexpr (Extra::kMode == 2) {
      // ---------------------------------------------------- reduce the tiles this rank owns (see ScatterC)
      const int tpr = extra.rows_per_rank / GEMM_BM;
      const int owned = tpr * tiles_n;
      const uint32_t* my_flags = extra.flags[extra.rank];
      constexpr int VEC = BN / 8;        // 16-byte vectors per tile row
      constexpr int RPI = 32 / VEC;      // rows handled per warp iteration (1 for BN = 256, 2 for BN = 128)
      bool ok2 = (*cta_abort == 0);
      for (int t = blockIdx.x; t < owned && ok2; t += gridDim.x) {
        if (lane < extra.world) {
          const uint32_t* f = my_flags + (static_cast<size_t>(t) * extra.world + lane) * 4 + q;
          const unsigned long long t0 = globaltimer_ns();
          uint32_t it = 0;
          while (static_cast<int32_t>(ld_acquire_sys_u32(f) - extra.epoch) < 0) {
            if ((++it & 0x3f) == 0 && (*cta_abort || globaltimer_ns() - t0 > extra.limit_ns)) {
              if (status) atomicCAS(status, 0, ERR_WAIT_PEER | (lane << 8));
              *cta_abort = 1;
              ok2 = false;
              break;
            }
          }
        }
        ok2 = __all_sync(0xffffffffu, ok2);
        if (!ok2) break;
        const int row_base = (t / tiles_n) * GEMM_BM + q * 32;
        const int col = (t % tiles_n) * BN + (lane % VEC) * 8;
        if (col < N) {
          constexpr int UNR = 4;  // rows in flight per lane
          for (int rr0 = lane / VEC; rr0 < 32; rr0 += RPI * UNR) {
            float acc[UNR][8];
#pragma unroll
            for (int j = 0; j < UNR; ++j)
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
            for (int r = 0; r < extra.world; ++r) {
              uint4 u[UNR];
#pragma unroll
              for (int j = 0; j < UNR; ++j) {
                const int row = row_base + rr0 + j * RPI;
                u[j] = (rr0 + j * RPI < 32) ? *reinterpret_cast<const uint4*>(extra.recv + (static_cast<size_t>(r) * extra.rows_per_rank + row) * N + col)
                                            : make_uint4(0, 0, 0, 0);
              }
#pragma unroll
              for (int j = 0; j < UNR; ++j) {
                const float2 a0 = unpack_bf16x2(u[j].x), a1 = unpack_bf16x2(u[j].y), a2 = unpack_bf16x2(u[j].z), a3 = unpack_bf16x2(u[j].w);
                acc[j][0] += a0.x; acc[j][1] += a0.y; acc[j][2] += a1.x; acc[j][3] += a1.y;
                acc[j][4] += a2.x; acc[j][5] += a2.y; acc[j][6] += a3.x; acc[j][7] += a3.y;
              }
            }
#pragma unroll
            for (int j = 0; j < UNR; ++j) {
              if (rr0 + j * RPI >= 32) break;
              uint4 o;
              o.x = pack_bf16x2(acc[j][0], acc[j][1]);
              o.y = pack_bf16x2(acc[j][2], acc[j][3]);
              o.z = pack_bf16x2(acc[j][4], acc[j][5]);
              o.w = pack_bf16x2(acc[j][6], acc[j][7]);
              *reinterpret_cast<uint4*>(extra.out + static_cast<size_t>(row_base + rr0 + j * RPI) * extra.ld_out + col) = o;
            }
          }
        }
      }
    }
  }
  if constexpr (Extra::kMode == 1) {
    if (warp >= 6) {
      // ---------------------------------------------------- gather warps: pull the peers' shards into `gathered`
      const int per_shard = extra.rows_per_rank / GATHER_PIECE_ROWS;
      const int total = (extra.world - 1) * per_shard;
      const int n16 = GATHER_PIECE_ROWS * extra.row_bytes / 16;  // 16-byte vectors per piece (rows are contiguous)
      for (int p = blockIdx.x * GATHER_WARPS + (warp - 6); p < total; p += gridDim.x * GATHER_WARPS) {
        const int s = p / per_shard, piece = p - s * per_shard;
        const int src = (extra.rank + 1 + s) % extra.world;  // nearest peer first: the order the tiles are walked in
        const size_t row0 = static_cast<size_t>(piece) * GATHER_PIECE_ROWS;
        const uint4* from = reinterpret_cast<const uint4*>(static_cast<const char*>(extra.peer[src]) + row0 * extra.row_bytes);
        uint4* to = reinterpret_cast<uint4*>(static_cast<char*>(extra.gathered) +
                                             (static_cast<size_t>(src) * extra.rows_per_rank + row0) * extra.row_bytes);
        for (int i = lane; i < n16; i += 32 * 8) {
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (i + u * 32 < n16) v[u] = from[i + u * 32];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (i + u * 32 < n16) to[i + u * 32] = v[u];
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(extra.counters + (src * extra.rows_per_rank + static_cast<int>(row0)) / GEMM_BM, 1u);
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    // give copies that are still in flight a bounded time to land before the smem goes away
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, NCOLS);
}

template <int BN, int STAGES, bool A_MN, bool B_MN, bool OUT_F32, bool TMA_EPI, typename Extra = NoExtra>
static cudaError_t launch_gemm(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                               int ldb, int ldc, int accumulate, int* status, int num_sms, cudaStream_t stream,
                               const int* tile_boff = nullptr, int b_stack_rows = 0, const Extra& extra = Extra()) {
  using S = GemmSmem<BN, STAGES>;
  // K-major operand: tensor [rows = M or N, cols = K], box [rows_tile, 64].
  // MN-major operand: tensor [rows = K, cols = M or N], box [64 k-rows, 64 cols].
  CUtensorMap tmA = A_MN ? make_tmap_2d(A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, size_t(lda) * 2, 64, 64,
                                        CU_TENSOR_MAP_SWIZZLE_128B)
                         : make_tmap_2d(A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, size_t(lda) * 2, GEMM_BM, GEMM_BK,
                                        CU_TENSOR_MAP_SWIZZLE_128B);
  // grouped: the map covers the whole stack (b_stack_rows rows), the kernel adds the expert's row offset
  const int b_rows = b_stack_rows > 0 ? b_stack_rows : (B_MN ? K : N);
  CUtensorMap tmB = B_MN ? make_tmap_2d(B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b_rows, N, size_t(ldb) * 2, 64, 64,
                                        CU_TENSOR_MAP_SWIZZLE_128B)
                         : make_tmap_2d(B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b_rows, K, size_t(ldb) * 2, BN, GEMM_BK,
                                        CU_TENSOR_MAP_SWIZZLE_128B);
  CUtensorMap tmC = tmA;  // placeholder when the direct-store epilogue is used
  if constexpr (TMA_EPI) {
    tmC = OUT_F32 ? make_tmap_2d(C, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, size_t(ldc) * 4, 32, 32,
                                 CU_TENSOR_MAP_SWIZZLE_128B)
                  : make_tmap_2d(C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, size_t(ldc) * 2, 32, 64,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
  }
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, OUT_F32, TMA_EPI, Extra>;
  if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), S::TOTAL); e != cudaSuccess) {
    set_last_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    return e;
  }
  const int splitk = (accumulate >> 8) > 1 ? (accumulate >> 8) : 1;
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN) * splitk;
  int grid = tiles < num_sms ? tiles : num_sms;
  if (Extra::kMode != 0) grid = num_sms;  // the collective's own work (gather pieces, owned tiles) is striped over every CTA
  constexpr int threads = Extra::kMode == 1 ? GEMM_THREADS + 32 * GATHER_WARPS : GEMM_THREADS;  // + the gather warps
  cudaError_t le = launch_pdl(kern, dim3(grid), dim3(threads), S::TOTAL, stream, tmA, tmB, tmC, C,
                              reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K, ldc, accumulate, status, tile_boff, extra);
  if (le != cudaSuccess) set_last_error(std::string("gemm launch: ") + cudaGetErrorString(le));
  return le;
}

template <int BN, int STAGES, bool TMA_EPI>
static cudaError_t dispatch_layout(bool a_mn, bool b_mn, bool out_f32, const void* A, const void* B, void* C,
                                   const void* bias, int M, int N, int K, int lda, int ldb, int ldc, int accumulate,
                                   int* status, int num_sms, cudaStream_t stream, const int* tile_boff = nullptr,
                                   int b_stack_rows = 0) {
#define SB_CASE(AM, BMN, OF)                                                                                       \
  if (a_mn == AM && b_mn == BMN && out_f32 == OF)                                                                  \
    return launch_gemm<BN, STAGES, AM, BMN, OF, TMA_EPI>(A, B, C, bias, M, N, K, lda, ldb, ldc, accumulate, status, \
                                                         num_sms, stream, tile_boff, b_stack_rows);
  SB_CASE(false, false, false)
  SB_CASE(false, false, true)
  SB_CASE(false, true, false)
  SB_CASE(false, true, true)
  SB_CASE(true, false, false)
  SB_CASE(true, false, true)
  SB_CASE(true, true, false)
  SB_CASE(true, true, true)
#undef SB_CASE
  return cudaErrorInvalidValue;
}

}  // namespace sb

// C ABI. Leading dimensions are in elements. Returns a cudaError_t value (0 = ok); sb_last_error() has details.
//   a_mn = 0: A is row-major [M, K] (pitch lda);  a_mn = 1: A is stored [K, M] (pitch lda)
//   b_mn = 0: B is row-major [N, K] (pitch ldb);  b_mn = 1: B is stored [K, N] (pitch ldb)
// Requirements: A/B base pointers 16-byte aligned, lda/ldb multiples of 8 elements.
// `status` is a device int that receives a non-zero code if a bounded wait expired.
// `splitk` > 1 cuts K into that many slices whose partial products are summed into C by TMA reduce-add: C must then be
// fp32, 16-byte aligned, and either zeroed by the caller or meant to be accumulated into (accumulate = 1).
extern "C" int sb_gemm_bf16_splitk(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                                   int ldb, int ldc, int a_mn, int b_mn, int out_f32, int accumulate, int bn, int splitk,
                                   int* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const size_t c_elem = out_f32 ? 4 : 2;
  const bool tma_epi = (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (size_t(ldc) * c_elem) % 16 == 0 &&
                       !(accumulate && !out_f32);
  const int num_kb = (K + sb::GEMM_BK - 1) / sb::GEMM_BK;
  if (splitk > num_kb) splitk = num_kb;
  if (splitk > 1) {
    if (!tma_epi || !out_f32) {
      sb::set_last_error("sb_gemm_bf16_splitk: split-K needs an fp32 C with a 16-byte aligned base and pitch");
      return (int)cudaErrorInvalidValue;
    }
    const int kb_per = (num_kb + splitk - 1) / splitk;
    splitk = (num_kb + kb_per - 1) / kb_per;  // no empty slice
  }
  accumulate = (accumulate ? 1 : 0) | ((splitk > 1 ? splitk : 0) << 8);
  try {
    if (bn == 256) {
      if (tma_epi)
        return (int)sb::dispatch_layout<256, 4, true>(a_mn != 0, b_mn != 0, out_f32 != 0, A, B, C, bias, M, N, K, lda, ldb,
                                                      ldc, accumulate, status, num_sms, stream);
      return (int)sb::dispatch_layout<256, 4, false>(a_mn != 0, b_mn != 0, out_f32 != 0, A, B, C, bias, M, N, K, lda, ldb,
                                                     ldc, accumulate, status, num_sms, stream);
    }
    if (tma_epi)
      return (int)sb::dispatch_layout<128, 6, true>(a_mn != 0, b_mn != 0, out_f32 != 0, A, B, C, bias, M, N, K, lda, ldb,
                                                    ldc, accumulate, status, num_sms, stream);
    return (int)sb::dispatch_layout<128, 6, false>(a_mn != 0, b_mn != 0, out_f32 != 0, A, B, C, bias, M, N, K, lda, ldb,
                                                   ldc, accumulate, status, num_sms, stream);
  } catch (const std::exception& e) {
    sb::set_last_error(e.what());
    return (int)cudaErrorInvalidValue;
  }
}

// Grouped GEMM over experts (M-contiguous layout): A [M, K] row-major holds the tokens sorted by expert, each expert's
// segment starting at a multiple of 128 rows (the tail of a segment is padding); B is the experts' weights stacked,
// [E * N, K] row-major (b_mn = 0, C = A * W_e^T) or [E * K, N] (b_mn = 1, C = A * W_e); tile_boff[t] (device, one int
// per 128-row tile of A) is the first row of that tile's expert in the stack: e * N, resp. e * K. C [M, N] bf16 or fp32.
// With b_mn = 1, K must be a multiple of 64 (a K tail would read the next expert's rows).
extern "C" int sb_gemm_bf16_grouped(const void* A, const void* B, void* C, const int* tile_boff, int M, int N, int K,
                                    int num_experts, int lda, int ldb, int ldc, int b_mn, int out_f32, int bn, int* status,
                                    int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (tile_boff == nullptr || num_experts <= 0 || (b_mn && K % sb::GEMM_BK != 0)) {
    sb::set_last_error("sb_gemm_bf16_grouped: needs tile_boff, num_experts > 0, and K % 64 == 0 when b_mn");
    return (int)cudaErrorInvalidValue;
  }
  const size_t c_elem = out_f32 ? 4 : 2;
  const bool tma_epi = (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (size_t(ldc) * c_elem) % 16 == 0;
  const int stack_rows = num_experts * (b_mn ? K : N);
  try {
    if (bn == 256) {
      if (tma_epi)
        return (int)sb::dispatch_layout<256, 4, true>(false, b_mn != 0, out_f32 != 0, A, B, C, nullptr, M, N, K, lda, ldb, ldc,
                                                      0, status, num_sms, stream, tile_boff, stack_rows);
      return (int)sb::dispatch_layout<256, 4, false>(false, b_mn != 0, out_f32 != 0, A, B, C, nullptr, M, N, K, lda, ldb, ldc,
                                                     0, status, num_sms, stream, tile_boff, stack_rows);
    }
    if (tma_epi)
      return (int)sb::dispatch_layout<128, 6, true>(false, b_mn != 0, out_f32 != 0, A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0,
                                                    status, num_sms, stream, tile_boff, stack_rows);
    return (int)sb::dispatch_layout<128, 6, false>(false, b_mn != 0, out_f32 != 0, A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0,
                                                   status, num_sms, stream, tile_boff, stack_rows);
  } catch (const std::exception& e) {
    sb::set_last_error(e.what());
    return (int)cudaErrorInvalidValue;
  }
}

// All-gather fused into the GEMM (see GatherA): C[M, N] = gathered * op(B) (+ bias), M = world * rows_per_rank.
// peers[r]: rank r's shard [rows_per_rank, K] bf16 with contiguous rows, as mapped into this GPU (own included; the own
// shard is not read). gathered: this GPU's [M, K] bf16 buffer whose rows of THIS rank the caller has already filled;
// counters: M / 128 words, zero before the first call; target = 32 * (number of calls made with these counters,
// this one included). rows_per_rank a multiple of 128, K a multiple of 8. B: [N, K] (b_mn = 0) or [K, N] (b_mn = 1).
// The caller makes sure (barrier) that every rank's shard is complete before the launch and stays until it ends.
extern "C" int sb_gemm_bf16_gather_a(const void* const* peers, int world, int rank, int rows_per_rank, void* gathered,
                                     unsigned* counters, unsigned target, const void* B, void* C, const void* bias, int N,
                                     int K, int ldb, int ldc, int b_mn, int bn, int* status, int num_sms, cudaStream_t stream) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || rows_per_rank <= 0 || rows_per_rank % sb::GEMM_BM != 0 || (K & 7)) {
    sb::set_last_error("sb_gemm_bf16_gather_a: 1..8 ranks, rows_per_rank a positive multiple of 128, K a multiple of 8");
    return (int)cudaErrorInvalidValue;
  }
  const int M = world * rows_per_rank;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (size_t(ldc) * 2) % 16) {
    sb::set_last_error("sb_gemm_bf16_gather_a: C must be 16-byte aligned with a 16-byte-multiple pitch");
    return (int)cudaErrorInvalidValue;
  }
  try {
    sb::GatherA ex{};
    for (int r = 0; r < 8; ++r) ex.peer[r] = peers[r < world ? r : 0];
    ex.gathered = gathered;
    ex.counters = counters;
    ex.target = target;
    ex.rows_per_rank = rows_per_rank;
    ex.world = world;
    ex.rank = rank;
    ex.row_bytes = K * 2;
    ex.limit_ns = sb::peer_wait_limit_ns();
#define SB_GA(BNV, ST, BM_)                                                                                                  \
  return (int)sb::launch_gemm<BNV, ST, false, BM_, false, true, sb::GatherA>(gathered, B, C, bias, M, N, K, K, ldb, ldc, 0, status, \
                                                                             num_sms, stream, nullptr, 0, ex);
    if (bn == 256) {
      if (b_mn) { SB_GA(256, 4, true) } else { SB_GA(256, 4, false) }
    }
    if (b_mn) { SB_GA(128, 6, true) } else { SB_GA(128, 6, false) }
#undef SB_GA
  } catch (const std::exception& e) {
    sb::set_last_error(e.what());
    return (int)cudaErrorInvalidValue;
  }
}

// Reduce-scatter fused into the GEMM (see ScatterC): out[rows_per_rank, N] = rows of THIS rank of sum_r (A_r * op(B_r)),
// every rank calling with its own A [M, K] and B, M = world * rows_per_rank. recv[o] / flags[o]: owner o's receive buffer
// ([world][rows_per_rank][N] bf16) and flag words ((rows_per_rank / 128) * ceil(N / bn) * world * 4, zero before the first
// call) as mapped into this GPU; epoch: 1, 2, 3, ... per call on a given pair of buffers. N a multiple of 8. The caller
// alternates between two receive buffers (a rank may run one call ahead of its peers).
extern "C" int sb_gemm_bf16_scatter_c(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int b_mn,
                                      const void* const* recv, const void* const* flags, int world, int rank, void* out,
                                      int ld_out, unsigned epoch, int bn, int* status, int num_sms, cudaStream_t stream) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || M <= 0 || M % (world * sb::GEMM_BM) != 0 || (N & 7)) {
    sb::set_last_error("sb_gemm_bf16_scatter_c: 1..8 ranks, M a multiple of world * 128, N a multiple of 8");
    return (int)cudaErrorInvalidValue;
  }
  const int rows_per_rank = M / world;
  try {
    sb::ScatterC ex{};
    for (int o = 0; o < 8; ++o) {
      const int src = o < world ? o : 0;
      ex.slot[o] = sb::make_tmap_2d(recv[src], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, size_t(world) * rows_per_rank, N, size_t(N) * 2,
                                    32, 64, CU_TENSOR_MAP_SWIZZLE_128B);
      ex.flags[o] = static_cast<uint32_t*>(const_cast<void*>(flags[src]));
    }
    ex.recv = static_cast<const __nv_bfloat16*>(recv[rank]);
    ex.out = static_cast<__nv_bfloat16*>(out);
    ex.ld_out = ld_out;
    ex.epoch = epoch;
    ex.rows_per_rank = rows_per_rank;
    ex.world = world;
    ex.rank = rank;
    ex.limit_ns = sb::peer_wait_limit_ns();
    void* c_unused = const_cast<void*>(recv[rank]);  // tmC is built but never stored through in this mode
#define SB_SC(BNV, ST, BM_)                                                                                                   \
  return (int)sb::launch_gemm<BNV, ST, false, BM_, false, true, sb::ScatterC>(A, B, c_unused, nullptr, M, N, K, lda, ldb, N, 0, status, \
                                                                              num_sms, stream, nullptr, 0, ex);
    if (bn == 256) {
      if (b_mn) { SB_SC(256, 4, true) } else { SB_SC(256, 4, false) }
    }
    if (b_mn) { SB_SC(128, 6, true) } else { SB_SC(128, 6, false) }
#undef SB_SC
  } catch (const std::exception& e) {
    sb::set_last_error(e.what());
    return (int)cudaErrorInvalidValue;
  }
}

extern "C" const char* sb_last_error() { return sb::last_error_buf(); }

extern "C" int sb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                            int ldb, int ldc, int a_mn, int b_mn, int out_f32, int accumulate, int bn, int* status,
                            int num_sms, cudaStream_t stream) {
  return sb_gemm_bf16_splitk(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_f32, accumulate, bn, 1, status, num_sms,
                             stream);
}

// 1: kernels of this library are launched with programmatic dependent launch (default); 0: plain stream order.
extern "C" void sb_set_pdl(int enabled) { sb::pdl_enabled() = enabled ? 1 : 0; }
extern "C" int sb_get_pdl(void) { return sb::pdl_enabled(); }
