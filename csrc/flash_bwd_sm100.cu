// Varlen causal flash attention, backward, on the 5th-gen tensor cores (sm_100a). Same segment table as the forward
// (flash_fwd_sm100.cu): seg[s] = { q_off, q_len, k_off, k_len }, query i sees keys j <= (k_len - q_len) + i.
//
// Three launches, no atomics, fixed summation order (bitwise reproducible):
//
//   delta    D_i = sum_d dO[i, d] * O[i, d]                                   one warp per (token, head)
//   dkv      one CTA per (128-key tile, kv head): K, V stay in shared memory; the query blocks (64 rows) of every query
//            head of the group that can see the tile stream through a 2-stage ring:
//                S^T  = K Q^T          dP^T = V dO^T                (M 128 keys, N 64 queries, K D)     -> TMEM
//                P^T  = 2^(S^T c - lse),   dS^T = P^T (dP^T - D) scale                      registers -> smem
//                dV  += P^T dO         dK  += dS^T Q                (M 128 keys, N D, K 64)   accumulated in TMEM
//   dq       one CTA per (128-query tile, query head): Q, dO stay in shared memory, key blocks (64) stream:
//                S = Q K^T, dP = dO V^T (M 128, N 64, K D);  dS = P (dP - D) scale;  dQ += dS K  (M 128, N D, K 64)
//
// The score products are recomputed in both passes (7 tile products instead of 5); in exchange every output tile has
// one owner, so nothing is accumulated through global memory. A Q / dO (or K / V) block is loaded once by TMA and used
// twice: K-major as the B operand of the score products and MN-major as the B operand of the gradient products.
// CTA = 10 warps: TMA producer, MMA issuer, 8 element-wise warps (two per TMEM lane quarter, 32 columns each).
// All mbarrier waits are bounded; on expiry the CTA records a status word, drains and frees its TMEM.
#include "common.cuh"

namespace sb {

constexpr int FB_T = 128;        // stationary tile rows (keys in dkv, queries in dq) = TMEM lanes
constexpr int FB_S = 64;         // streamed block rows
constexpr int FB_THREADS = 320;  // TMA warp, MMA warp, 8 element-wise warps
constexpr int FB_STAGES = 2;

template <int D>
struct FbSmem {
  static constexpr int NCH = D / 64;
  static constexpr int TILE_BYTES = FB_T * 128 * NCH;  // stationary operand, [NCH][128 rows][128 B]
  static constexpr int BLK_BYTES = FB_S * 128 * NCH;   // streamed operand, [NCH][64 rows][128 B]
  static constexpr int PDS_BYTES = FB_T * 128;         // [128 rows][64 bf16]: one 128-byte swizzle row per TMEM lane
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = 2 * TILE_BYTES + 2 * FB_STAGES * BLK_BYTES + 2 * PDS_BYTES + BAR_BYTES + 1024;
  static constexpr int TMEM_COLS = 512;  // scores: 2 x 64 @0, dP: 2 x 64 @128, accumulators @256 (and @256 + D)
};

__device__ __forceinline__ float fb_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void fb_named_barrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// -------------------------------------------------------------------------------------------------- delta
// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h).
__global__ void flash_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                       float* __restrict__ delta, int T, int H, int D, int o_stride, int do_stride,
                                       int delta_stride) {
  pdl_wait();
  pdl_launch_dependents();
  const long w = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long>(T) * H) return;
  const int t = static_cast<int>(w / H), h = static_cast<int>(w % H);
  const __nv_bfloat16* po = o + static_cast<size_t>(t) * o_stride + h * D;
  const __nv_bfloat16* pd = d_o + static_cast<size_t>(t) * do_stride + h * D;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(po + i));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pd + i));
    acc += a.x * b.x + a.y * b.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[static_cast<size_t>(h) * delta_stride + t] = acc;
}

// Shared skeleton of the two passes. PASS_DQ = false: stationary = (K, V) tile, streamed = (Q, dO) blocks, outputs
// dK and dV. PASS_DQ = true: stationary = (Q, dO) tile, streamed = (K, V) blocks, output dQ.
//   tmA0 / tmA1: tensor maps of the two stationary operands (box 128 rows), tmB0 / tmB1: of the streamed ones (box 64).
//   score product 0:  A0 x B0^T  (K Q^T   or  Q K^T)      score product 1:  A1 x B1^T  (V dO^T  or  dO V^T)
//   dkv: acc0 (dV) += P^T  x B1 (dO),  acc1 (dK) += dS^T x B0 (Q)          dq: acc0 (dQ) += dS x B0 (K)
template <int D, bool PASS_DQ>
__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                 const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
                 const float* __restrict__ lse, const float* __restrict__ delta, __nv_bfloat16* __restrict__ out0,
                 __nv_bfloat16* __restrict__ out1, const int* __restrict__ seg, int nseg, int Hq, int Hkv, int out0_stride,
                 int out1_stride, int stat_stride, float scale, int* status) {
  using S = FbSmem<D>;
  constexpr int NCH = S::NCH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA0 = smem;
  uint8_t* sA1 = sA0 + S::TILE_BYTES;
  uint8_t* sB0 = sA1 + S::TILE_BYTES;                 // [FB_STAGES]
  uint8_t* sB1 = sB0 + FB_STAGES * S::BLK_BYTES;      // [FB_STAGES]
  uint8_t* sP = sB1 + FB_STAGES * S::BLK_BYTES;       // P^T (dkv only)
  uint8_t* sDS = sP + S::PDS_BYTES;                   // dS^T or dS
  uint64_t* a_full = reinterpret_cast<uint64_t*>(sDS + S::PDS_BYTES);
  uint64_t* b_full = a_full + 1;              // [2]
  uint64_t* b_empty = b_full + FB_STAGES;     // [2]
  uint64_t* sc_full = b_empty + FB_STAGES;    // [2] both score products of a block are in TMEM
  uint64_t* pds_full = sc_full + 2;           // element-wise warps -> MMA: P / dS are in shared memory (8 arrivals)
  uint64_t* pds_free = pds_full + 1;          // MMA -> element-wise: the gradient products have read them
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pds_free + 1);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* work = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = Hq / Hkv;
  const int hy = blockIdx.y;  // kv head (dkv) or query head (dq)

  if (threadIdx.x == 0) {
    mbar_init(a_full, 1);
    for (int s = 0; s < FB_STAGES; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&b_empty[s], 1);
    }
    mbar_init(&sc_full[0], 1);
    mbar_init(&sc_full[1], 1);
    mbar_init(pds_full, 8);
    mbar_init(pds_free, 1);
    *cta_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA0);
    tma_prefetch_desc(&tmA1);
    tma_prefetch_desc(&tmB0);
    tma_prefetch_desc(&tmB1);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, S::TMEM_COLS);
    tmem_relinquish();
  }
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    int t = blockIdx.x, found = -1, tile = 0;
    for (int s = 0; s < nseg; ++s) {
      const int len = PASS_DQ ? seg[4 * s + 1] : seg[4 * s + 3];
      const int nt = (len + FB_T - 1) / FB_T;
      if (t < nt) {
        found = s;
        tile = t;
        break;
      }
      t -= nt;
    }
    work[0] = found;
    work[1] = tile;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int sidx = work[0];
  if (sidx >= 0) {
    const int q_off = seg[4 * sidx], q_len = seg[4 * sidx + 1], k_off = seg[4 * sidx + 2], k_len = seg[4 * sidx + 3];
    const int shift = k_len - q_len;
    const int t0 = work[1] * FB_T;  // first row of the stationary tile inside the segment
    // streamed blocks [blk_lo, blk_hi) per query head; heads: dkv loops over the G heads of the group, dq has one
    int blk_lo, blk_hi, n_heads;
    if (PASS_DQ) {
      blk_lo = 0;
      blk_hi = (min(k_len, shift + t0 + FB_T) + FB_S - 1) / FB_S;
      n_heads = 1;
    } else {
      blk_lo = max(0, t0 - shift) / FB_S;
      blk_hi = (q_len + FB_S - 1) / FB_S;
      n_heads = G;
    }
    const int per_head = blk_hi - blk_lo;
    const int n_it = per_head * n_heads;
    const int a_col = hy * D;                            // column of the stationary operand's head
    const int a_row = (PASS_DQ ? q_off : k_off) + t0;
    const int b_row0 = PASS_DQ ? k_off : q_off;

    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        mbar_arrive_expect_tx(a_full, 2 * S::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tma_load_2d(sA0 + c * (FB_T * 128), &tmA0, a_full, a_col + c * 64, a_row);
          tma_load_2d(sA1 + c * (FB_T * 128), &tmA1, a_full, a_col + c * 64, a_row);
        }
        for (int it = 0; it < n_it; ++it) {
          const int st = it % FB_STAGES;
          if (!mbar_wait(&b_empty[st], ((it / FB_STAGES) & 1) ^ 1, cta_abort, status, ERR_WAIT_EMPTY)) break;
          const int hd = it / per_head, blk = blk_lo + it % per_head;
          const int b_col = (PASS_DQ ? hy / G : hy * G + hd) * D;
          mbar_arrive_expect_tx(&b_full[st], 2 * S::BLK_BYTES);
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            tma_load_2d(sB0 + st * S::BLK_BYTES + c * (FB_S * 128), &tmB0, &b_full[st], b_col + c * 64, b_row0 + blk * FB_S);
            tma_load_2d(sB1 + st * S::BLK_BYTES + c * (FB_S * 128), &tmB1, &b_full[st], b_col + c * 64, b_row0 + blk * FB_S);
          }
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc_sc = make_idesc(FB_T, FB_S, 1, 1, 0, 0);  // scores: both operands K-major
        constexpr uint32_t idesc_g = make_idesc(FB_T, D, 1, 1, 0, 1);      // gradients: B (streamed block) MN-major
        const uint32_t a0 = smem_u32(sA0), a1 = smem_u32(sA1), p_addr = smem_u32(sP), ds_addr = smem_u32(sDS);
        auto issue_scores = [&](int it) {
          const uint32_t b0 = smem_u32(sB0 + (it % FB_STAGES) * S::BLK_BYTES), b1 = smem_u32(sB1 + (it % FB_STAGES) * S::BLK_BYTES);
          const uint32_t buf = (it & 1) * FB_S;
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t oa = (k >> 2) * (FB_T * 128) + (k & 3) * 32, ob = (k >> 2) * (FB_S * 128) + (k & 3) * 32;
            umma_f16(tmem_base + buf, make_smem_desc(a0 + oa, 16, 1024, UMMA_SWIZZLE_128B),
                     make_smem_desc(b0 + ob, 16, 1024, UMMA_SWIZZLE_128B), idesc_sc, k != 0 ? 1u : 0u);
          }
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t oa = (k >> 2) * (FB_T * 128) + (k & 3) * 32, ob = (k >> 2) * (FB_S * 128) + (k & 3) * 32;
            umma_f16(tmem_base + 128 + buf, make_smem_desc(a1 + oa, 16, 1024, UMMA_SWIZZLE_128B),
                     make_smem_desc(b1 + ob, 16, 1024, UMMA_SWIZZLE_128B), idesc_sc, k != 0 ? 1u : 0u);
          }
          umma_commit(&sc_full[it & 1]);
        };
        bool ok = mbar_wait(a_full, 0, cta_abort, status, ERR_WAIT_FULL) &&
                  mbar_wait(&b_full[0], 0, cta_abort, status, ERR_WAIT_FULL);
        if (ok) {
          tc_fence_after();
          issue_scores(0);
        }
        for (int it = 0; it < n_it && ok; ++it) {
          if (it + 1 < n_it) {
            ok = mbar_wait(&b_full[(it + 1) % FB_STAGES], ((it + 1) / FB_STAGES) & 1, cta_abort, status, ERR_WAIT_FULL);
            if (!ok) break;
            tc_fence_after();
            issue_scores(it + 1);
          }
          ok = mbar_wait(pds_full, it & 1, cta_abort, status, ERR_WAIT_TMEM_EMPTY);
          if (!ok) break;
          tc_fence_after();
          const uint32_t b0 = smem_u32(sB0 + (it % FB_STAGES) * S::BLK_BYTES), b1 = smem_u32(sB1 + (it % FB_STAGES) * S::BLK_BYTES);
#pragma unroll
          for (int k = 0; k < FB_S / 16; ++k) {
            // A: one 128-byte row per lane, 16 elements = 32 B; B: streamed block read MN-major, 16 rows = 2048 B,
            // 64-wide chunks of the head dim FB_S * 128 B apart
            if (!PASS_DQ)
              umma_f16(tmem_base + 256, make_smem_desc(p_addr + k * 32, 16, 1024, UMMA_SWIZZLE_128B),
                       make_smem_desc(b1 + k * 2048, FB_S * 128, 1024, UMMA_SWIZZLE_128B), idesc_g, (it != 0 || k != 0) ? 1u : 0u);
            umma_f16(tmem_base + 256 + (PASS_DQ ? 0 : D), make_smem_desc(ds_addr + k * 32, 16, 1024, UMMA_SWIZZLE_128B),
                     make_smem_desc(b0 + k * 2048, FB_S * 128, 1024, UMMA_SWIZZLE_128B), idesc_g, (it != 0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&b_empty[it % FB_STAGES]);
          umma_commit(pds_free);
        }
      }
    } else {
      // ------------------------------------------------------------------ element-wise warps
      const int quarter = warp & 3, half = (warp - 2) >> 2;
      const int row = quarter * 32 + lane;  // TMEM lane: key (dkv) or query (dq) inside the tile
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const float c_log2 = scale * 1.4426950408889634f;
      const int ti = t0 + row;  // index inside the segment of this thread's key / query
      float my_lse2 = 0.f, my_delta = 0.f;
      if (PASS_DQ) {
        const bool v = ti < q_len;
        my_lse2 = v ? lse[static_cast<size_t>(hy) * stat_stride + q_off + ti] * 1.4426950408889634f : INFINITY;
        my_delta = v ? delta[static_cast<size_t>(hy) * stat_stride + q_off + ti] : 0.f;
      }
      bool ok = true;
      for (int it = 0; it < n_it; ++it) {
        const int hd = it / per_head, blk = blk_lo + it % per_head;
        const int c0 = blk * FB_S + half * 32;  // first streamed index (query in dkv, key in dq) of this warp's columns
        float col_lse2 = 0.f, col_delta = 0.f;
        if (!PASS_DQ) {
          // lane l fetches the statistics of query c0 + l; column c's values are taken by shuffle below
          const int qi = c0 + lane;
          const int hq = hy * G + hd;
          const bool v = qi < q_len;
          col_lse2 = v ? lse[static_cast<size_t>(hq) * stat_stride + q_off + qi] * 1.4426950408889634f : INFINITY;
          col_delta = v ? delta[static_cast<size_t>(hq) * stat_stride + q_off + qi] : 0.f;
        }
        ok = mbar_wait(&sc_full[it & 1], (it >> 1) & 1, cta_abort, status, ERR_WAIT_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t rs[32], rd[32];
        tmem_ld_32x32(lane_addr + (it & 1) * FB_S + half * 32, rs);
        tmem_ld_32x32(lane_addr + 128 + (it & 1) * FB_S + half * 32, rd);
        tmem_ld_wait();
        // visible columns. dkv: key ti (row) is seen by query c0 + c iff ti <= shift + c0 + c and ti < k_len.
        //                  dq:  query ti sees key c0 + c iff c0 + c <= shift + ti and c0 + c < k_len.
        int cmin, cmax;
        if (PASS_DQ) {
          cmin = 0;
          cmax = min(shift + ti, k_len - 1) - c0;
        } else {
          cmin = (ti < k_len) ? ti - shift - c0 : 64;
          cmax = 31;
        }
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float p[2], ds[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const float l2 = PASS_DQ ? my_lse2 : __shfl_sync(0xffffffffu, col_lse2, c + u);
            const float dl = PASS_DQ ? my_delta : __shfl_sync(0xffffffffu, col_delta, c + u);
            float pv = fb_exp2(fmaf(__uint_as_float(rs[c + u]), c_log2, -l2));
            if (c + u < cmin || c + u > cmax) pv = 0.f;
            p[u] = pv;
            ds[u] = pv * (__uint_as_float(rd[c + u]) - dl) * scale;
          }
          pk[c >> 1] = pack_bf16x2(p[0], p[1]);
          dk[c >> 1] = pack_bf16x2(ds[0], ds[1]);
        }
        if (it > 0) {
          ok = mbar_wait(pds_free, (it - 1) & 1, cta_abort, status, ERR_WAIT_TMEM_FULL);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        {
          const int sw = row & 7;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int ch = half * 4 + i;  // 16-byte chunk of the 128-byte row
            if (!PASS_DQ)
              *reinterpret_cast<uint4*>(sP + row * 128 + ((ch ^ sw) << 4)) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
            *reinterpret_cast<uint4*>(sDS + row * 128 + ((ch ^ sw) << 4)) = make_uint4(dk[4 * i], dk[4 * i + 1], dk[4 * i + 2], dk[4 * i + 3]);
          }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(pds_full);
      }
      // ---- epilogue: accumulators -> bf16 -> staged through the streamed operands' buffers -> coalesced rows
      if (ok && n_it > 0) {
        ok = mbar_wait(pds_free, (n_it - 1) & 1, cta_abort, status, ERR_WAIT_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        constexpr int CH = D / 8;  // 16-byte chunks per output row
        constexpr int HALF_COLS = D / 2;
        const int n_acc = PASS_DQ ? 1 : 2;
        for (int a = 0; a < n_acc; ++a) {
          uint8_t* stage = (a == 0) ? sB1 : sB0;  // FB_STAGES * BLK_BYTES = 128 rows * D * 2 bytes
#pragma unroll
          for (int c4 = 0; c4 < HALF_COLS / 32; ++c4) {
            uint32_t r[32];
            const int col = half * HALF_COLS + c4 * 32;
            if (n_it > 0) {
              tmem_ld_32x32(lane_addr + 256 + a * D + col, r);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = 0;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1]));
              v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
              v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
              v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
              const int ch = col / 8 + i;
              *reinterpret_cast<uint4*>(stage + row * (D * 2) + ((ch ^ (row & (CH - 1))) << 4)) = v;
            }
          }
        }
        fb_named_barrier(1, 256);
        const int t = threadIdx.x - 64;  // 0..255
        const int rows_valid = min(FB_T, (PASS_DQ ? q_len : k_len) - t0);
        const int out_row0 = (PASS_DQ ? q_off : k_off) + t0;
        for (int a = 0; a < n_acc; ++a) {
          const uint8_t* stage = (a == 0) ? sB1 : sB0;
          __nv_bfloat16* dst = (a == 0) ? out0 : out1;
          const int stride = (a == 0) ? out0_stride : out1_stride;
          for (int idx = t; idx < rows_valid * CH; idx += 256) {
            const int rr = idx / CH, ch = idx % CH;
            const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * (D * 2) + ((ch ^ (rr & (CH - 1))) << 4));
            *reinterpret_cast<uint4*>(dst + static_cast<size_t>(out_row0 + rr) * stride + hy * D + ch * 8) = v;
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    const unsigned long long t_a = globaltimer_ns();
    while (globaltimer_ns() - t_a < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, S::TMEM_COLS);
}

template <int D>
static int launch_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                            float* delta, void* dq, void* dk, void* dv, const int* seg, int nseg, int max_q_tiles,
                            int max_k_tiles, int Tq, int Tk, int Hq, int Hkv, int q_stride, int k_stride, int v_stride,
                            int o_stride, int do_stride, int dq_stride, int dk_stride, int dv_stride, int stat_stride,
                            float scale, int* status, cudaStream_t s) {
  using S = FbSmem<D>;
  using bf16 = __nv_bfloat16;
  auto map = [&](const void* p, int rows, int heads, int stride, int box_rows) {
    return make_tmap_2d(p, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, size_t(heads) * D, size_t(stride) * 2, box_rows, 64,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  };
  {
    const long warps = static_cast<long>(Tq) * Hq;
    const int blocks = static_cast<int>((warps * 32 + 255) / 256);
    cudaError_t e = launch_pdl(flash_bwd_delta_kernel, dim3(blocks), dim3(256), 0, s, (const bf16*)o, (const bf16*)d_o, delta, Tq,
                               Hq, D, o_stride, do_stride, stat_stride);
    if (e != cudaSuccess) return (int)e;
  }
  {
    auto kern = flash_bwd_kernel<D, false>;
    if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), S::TOTAL); e != cudaSuccess) return (int)e;
    cudaError_t e = launch_pdl(kern, dim3(max_k_tiles, Hkv), dim3(FB_THREADS), S::TOTAL, s, map(k, Tk, Hkv, k_stride, FB_T),
                               map(v, Tk, Hkv, v_stride, FB_T), map(q, Tq, Hq, q_stride, FB_S), map(d_o, Tq, Hq, do_stride, FB_S),
                               lse, (const float*)delta, (bf16*)dv, (bf16*)dk, seg, nseg, Hq, Hkv, dv_stride, dk_stride,
                               stat_stride, scale, status);
    if (e != cudaSuccess) return (int)e;
  }
  {
    auto kern = flash_bwd_kernel<D, true>;
    if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), S::TOTAL); e != cudaSuccess) return (int)e;
    cudaError_t e = launch_pdl(kern, dim3(max_q_tiles, Hq), dim3(FB_THREADS), S::TOTAL, s, map(q, Tq, Hq, q_stride, FB_T),
                               map(d_o, Tq, Hq, do_stride, FB_T), map(k, Tk, Hkv, k_stride, FB_S), map(v, Tk, Hkv, v_stride, FB_S),
                               lse, (const float*)delta, (bf16*)dq, (bf16*)nullptr, seg, nseg, Hq, Hkv, dq_stride, 0, stat_stride,
                               scale, status);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

}  // namespace sb

// Gradients of sb_flash_fwd. q / k / v / o / d_o as in the forward (o, d_o: [Tq, Hq * D] with their pitches); lse: the
// forward's [Hq, stat_stride]; delta: scratch of the same shape; dq: [Tq, Hq, D] (pitch dq_stride), dk / dv: [Tk, Hkv, D].
// Rows of dq / dk / dv outside every segment are left untouched. max_q_tiles / max_k_tiles: upper bounds of the number of
// 128-row tiles over all segments on the query and on the key side.
extern "C" int sb_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                            float* delta, void* dq, void* dk, void* dv, const int* seg, int nseg, int max_q_tiles,
                            int max_k_tiles, int Tq, int Tk, int Hq, int Hkv, int D, int q_stride, int k_stride, int v_stride,
                            int o_stride, int do_stride, int dq_stride, int dk_stride, int dv_stride, int stat_stride,
                            float scale, int* status, cudaStream_t s) {
  if (nseg <= 0 || Tq <= 0 || Tk <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0) return (int)cudaErrorInvalidValue;
  try {
    if (D == 64)
      return sb::launch_flash_bwd<64>(q, k, v, o, d_o, lse, delta, dq, dk, dv, seg, nseg, max_q_tiles, max_k_tiles, Tq, Tk, Hq,
                                      Hkv, q_stride, k_stride, v_stride, o_stride, do_stride, dq_stride, dk_stride, dv_stride,
                                      stat_stride, scale, status, s);
    if (D == 128)
      return sb::launch_flash_bwd<128>(q, k, v, o, d_o, lse, delta, dq, dk, dv, seg, nseg, max_q_tiles, max_k_tiles, Tq, Tk, Hq,
                                       Hkv, q_stride, k_stride, v_stride, o_stride, do_stride, dq_stride, dk_stride, dv_stride,
                                       stat_stride, scale, status, s);
  } catch (const std::exception& e) {
    sb::set_last_error(e.what());
    return (int)cudaErrorInvalidValue;
  }
  return -1;
}
