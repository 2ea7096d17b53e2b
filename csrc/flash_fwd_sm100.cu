// Varlen causal flash attention, forward, on the 5th-gen tensor cores (sm_100a). Training, prefill and
// context-parallel attention all go through this kernel: the work is described by a table of SEGMENTS
//
//     seg[s] = { q_off, q_len, k_off, k_len }        rows [q_off, q_off + q_len) of Q attend rows [k_off, k_off + k_len)
//                                                    of K / V, causally aligned at the end: query i sees keys
//                                                    j <= (k_len - q_len) + i   (k_len >= q_len)
//
// so a packed training batch is one segment per sequence with q_off = k_off, a prefill over a cached prefix has
// k_len > q_len, and a context-parallel rank passes its local query chunk against a prefix of the gathered keys.
// GQA: query head h uses kv head h / (Hq / Hkv).
//
// One CTA = one 128-row query tile of one head. 6 warps: warp 0 issues TMA loads (Q once, K / V tiles of 128 keys
// through a 2-stage ring), warp 1 owns TMEM and issues tcgen05.mma, warps 2-5 are the softmax: thread r owns query row
// r (= TMEM lane r).
//
//   S_j  = Q K_j^T            M 128, N 128, K D        TMEM, two buffers: S_{j+1} is issued before the softmax of tile j
//   P_j  = 2^(S_j*c - m)      registers -> bf16 -> shared memory (128B-swizzled, the A operand of the next product)
//   O   += P_j V_j            M 128, N D,  K 128       accumulated in TMEM over all tiles of the row
//
// The running maximum m is only raised when a tile exceeds it by more than 2^8 (decided per warp): otherwise the stale
// maximum keeps being used, p stays below 256 and O needs no correction; when it is raised the owning thread rescales
// its O row in TMEM (tcgen05.ld / st) before the next product is issued. Scores live in the log2 domain.
// out = O / l as bf16, lse = ln(sum exp(s * scale)) per row (fp32), both written only for rows inside the segment.
// Every mbarrier wait is bounded: on expiry the CTA records a status word, drains and returns with its TMEM freed.
#include "common.cuh"

namespace sb {

constexpr int FA_BM = 128;       // query rows per CTA
constexpr int FA_BN = 128;       // keys per tile
constexpr int FA_THREADS = 192;  // TMA warp, MMA warp, 4 softmax warps
constexpr int FA_KV_STAGES = 2;

template <int D>
struct FaSmem {
  static constexpr int NCH = D / 64;                  // 128-byte chunks of the head dim
  static constexpr int Q_BYTES = FA_BM * 128 * NCH;   // [NCH][128 rows][128 B]
  static constexpr int KV_BYTES = FA_BN * 128 * NCH;  // one K or V tile
  static constexpr int P_BYTES = FA_BM * FA_BN * 2;   // [2 chunks of 64 keys][128 rows][128 B]
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = Q_BYTES + 2 * FA_KV_STAGES * KV_BYTES + P_BYTES + BAR_BYTES + 1024;  // +1024: alignment
  static constexpr int TMEM_COLS = 512;  // S0 @0, S1 @128, O @256 (D columns)
};

__device__ __forceinline__ float fa_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ void fa_named_barrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                 const int* __restrict__ seg, int nseg, int Hq, int Hkv, int out_stride, int lse_stride, float scale,
                 int* status) {
  using S = FaSmem<D>;
  constexpr int NCH = S::NCH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + S::Q_BYTES;
  uint8_t* sV = sK + FA_KV_STAGES * S::KV_BYTES;
  uint8_t* sP = sV + FA_KV_STAGES * S::KV_BYTES;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(sP + S::P_BYTES);
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + FA_KV_STAGES;
  uint64_t* v_full = k_empty + FA_KV_STAGES;
  uint64_t* v_empty = v_full + FA_KV_STAGES;
  uint64_t* s_full = v_empty + FA_KV_STAGES;  // [2]
  uint64_t* p_full = s_full + 2;
  uint64_t* o_done = p_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* work = reinterpret_cast<int*>(tmem_slot + 2);  // [0] segment or -1, [1] tile in segment

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int kvh = h / (Hq / Hkv);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FA_KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(p_full, 4);  // one arrival per softmax warp
    mbar_init(o_done, 1);
    *cta_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, S::TMEM_COLS);
    tmem_relinquish();
  }
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    // which (segment, tile) is this CTA's? Tiles are numbered segment by segment.
    int t = blockIdx.x, found = -1, tile = 0;
    for (int s = 0; s < nseg; ++s) {
      const int nt = (seg[4 * s + 1] + FA_BM - 1) / FA_BM;
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
    const int q0 = work[1] * FA_BM;              // first query row of this tile inside the segment
    const int shift = k_len - q_len;             // query i sees keys j <= shift + i
    const int kv_hi = min(k_len, shift + q0 + FA_BM);
    const int n_kv = (kv_hi + FA_BN - 1) / FA_BN;

    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        mbar_arrive_expect_tx(q_full, S::Q_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c) tma_load_2d(sQ + c * (FA_BM * 128), &tmQ, q_full, h * D + c * 64, q_off + q0);
        for (int j = 0; j < n_kv; ++j) {
          const int st = j % FA_KV_STAGES;
          const uint32_t par = (j / FA_KV_STAGES) & 1;
          if (!mbar_wait(&k_empty[st], par ^ 1, cta_abort, status, ERR_WAIT_EMPTY)) break;
          mbar_arrive_expect_tx(&k_full[st], S::KV_BYTES);
#pragma unroll
          for (int c = 0; c < NCH; ++c)
            tma_load_2d(sK + st * S::KV_BYTES + c * (FA_BN * 128), &tmK, &k_full[st], kvh * D + c * 64, k_off + j * FA_BN);
          if (!mbar_wait(&v_empty[st], par ^ 1, cta_abort, status, ERR_WAIT_EMPTY)) break;
          mbar_arrive_expect_tx(&v_full[st], S::KV_BYTES);
#pragma unroll
          for (int c = 0; c < NCH; ++c)
            tma_load_2d(sV + st * S::KV_BYTES + c * (FA_BN * 128), &tmV, &v_full[st], kvh * D + c * 64, k_off + j * FA_BN);
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc_s = make_idesc(FA_BM, FA_BN, 1, 1, 0, 0);
        constexpr uint32_t idesc_o = make_idesc(FA_BM, D, 1, 1, 0, 1);  // B = V read MN-major
        const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
        auto issue_s = [&](int j) {
          const uint32_t k_addr = smem_u32(sK + (j % FA_KV_STAGES) * S::KV_BYTES);
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t off = (k >> 2) * (FA_BM * 128) + (k & 3) * 32;
            umma_f16(tmem_base + (j & 1) * FA_BN, make_smem_desc(q_addr + off, 16, 1024, UMMA_SWIZZLE_128B),
                     make_smem_desc(k_addr + off, 16, 1024, UMMA_SWIZZLE_128B), idesc_s, k != 0 ? 1u : 0u);
          }
          umma_commit(&k_empty[j % FA_KV_STAGES]);
          umma_commit(&s_full[j & 1]);
        };
        bool ok = mbar_wait(q_full, 0, cta_abort, status, ERR_WAIT_FULL) &&
                  mbar_wait(&k_full[0], 0, cta_abort, status, ERR_WAIT_FULL);
        if (ok) {
          tc_fence_after();
          issue_s(0);
        }
        for (int j = 0; j < n_kv && ok; ++j) {
          if (j + 1 < n_kv) {
            // S_{j+1} goes to the other buffer (the softmax of tile j-1 has released it: its p_full was seen below)
            ok = mbar_wait(&k_full[(j + 1) % FA_KV_STAGES], ((j + 1) / FA_KV_STAGES) & 1, cta_abort, status, ERR_WAIT_FULL);
            if (!ok) break;
            tc_fence_after();
            issue_s(j + 1);
          }
          ok = mbar_wait(p_full, j & 1, cta_abort, status, ERR_WAIT_TMEM_EMPTY) &&
               mbar_wait(&v_full[j % FA_KV_STAGES], (j / FA_KV_STAGES) & 1, cta_abort, status, ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t v_addr = smem_u32(sV + (j % FA_KV_STAGES) * S::KV_BYTES);
#pragma unroll
          for (int k = 0; k < FA_BN / 16; ++k) {
            // A = P: K-major, 64-key chunks 16 KB apart; B = V tile [128 keys, D]: MN-major, 16 keys = 2048 B,
            // 64-wide chunks of the head dim FA_BN * 128 B apart
            const uint64_t da = make_smem_desc(p_addr + (k >> 2) * (FA_BM * 128) + (k & 3) * 32, 16, 1024, UMMA_SWIZZLE_128B);
            const uint64_t db = make_smem_desc(v_addr + k * 2048, FA_BN * 128, 1024, UMMA_SWIZZLE_128B);
            umma_f16(tmem_base + 2 * FA_BN, da, db, idesc_o, (j != 0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&v_empty[j % FA_KV_STAGES]);
          umma_commit(o_done);
        }
      }
    } else {
      // ------------------------------------------------------------------ softmax + epilogue
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;  // query row inside the tile = TMEM lane
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const float c_log2 = scale * 1.4426950408889634f;
      const int qi = q0 + row;
      const int my_limit = shift + qi;  // last key this row may see
      float m_run = -INFINITY, l_run = 0.f;
      bool ok = true;
      for (int j = 0; j < n_kv; ++j) {
        ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, cta_abort, status, ERR_WAIT_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t s_addr = lane_addr + (j & 1) * FA_BN;
        const int key0 = j * FA_BN;
        // a tile needs masking when it reaches past the diagonal of this CTA's first row or past the last key
        const bool masked = (key0 + FA_BN - 1 > shift + q0) || (key0 + FA_BN > k_len);
        const int lim = min(my_limit, k_len - 1) - key0;  // columns <= lim are visible to this row
        // ---- pass 1: row maximum
        float mx = -INFINITY;
#pragma unroll
        for (int c4 = 0; c4 < FA_BN / 32; ++c4) {
          uint32_t r[32];
          tmem_ld_32x32(s_addr + c4 * 32, r);
          tmem_ld_wait();
          if (masked) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c4 * 32 + i <= lim) mx = fmaxf(mx, __uint_as_float(r[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
          }
        }
        mx *= c_log2;  // scale > 0: the maximum commutes with the scaling
        const float m_new = fmaxf(m_run, mx);
        bool raise = false;
        if (j == 0) {
          m_run = (m_new == -INFINITY) ? 0.f : m_new;
        } else {
          raise = __any_sync(0xffffffffu, m_new > m_run + 8.f);
        }
        const float m_use = raise ? ((m_new == -INFINITY) ? 0.f : m_new) : m_run;
        // ---- pass 2: p = 2^(s*c - m), packed to bf16; the row sum uses the unrounded values
        uint32_t pk[FA_BN / 2];
        float lsum = 0.f;
#pragma unroll
        for (int c4 = 0; c4 < FA_BN / 32; ++c4) {
          uint32_t r[32];
          tmem_ld_32x32(s_addr + c4 * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = fa_exp2(fmaf(__uint_as_float(r[i]), c_log2, -m_use));
            float p1 = fa_exp2(fmaf(__uint_as_float(r[i + 1]), c_log2, -m_use));
            if (masked) {
              if (c4 * 32 + i > lim) p0 = 0.f;
              if (c4 * 32 + i + 1 > lim) p1 = 0.f;
            }
            lsum += p0 + p1;
            pk[c4 * 16 + (i >> 1)] = pack_bf16x2(p0, p1);
          }
        }
        // ---- the previous product has finished: P may be overwritten and O may be corrected
        if (j > 0) {
          ok = mbar_wait(o_done, (j - 1) & 1, cta_abort, status, ERR_WAIT_TMEM_FULL);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          if (raise) {
            const float f = fa_exp2(m_run - m_use);  // <= 1
            l_run *= f;
#pragma unroll
            for (int c4 = 0; c4 < D / 32; ++c4) {
              uint32_t r[32];
              tmem_ld_32x32(lane_addr + 2 * FA_BN + c4 * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
              tmem_st_32x32(lane_addr + 2 * FA_BN + c4 * 32, r);
            }
            tmem_st_wait();
            m_run = m_use;
          }
        }
        l_run += lsum;
        // ---- P -> shared memory, canonical K-major 128B-swizzle layout: 16-byte chunk i of row r sits at (i ^ (r % 8))
        {
          uint8_t* prow = sP + row * 128;
          const int sw = row & 7;
#pragma unroll
          for (int i = 0; i < FA_BN / 8; ++i) {
            uint4 v = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
            *reinterpret_cast<uint4*>(prow + (i >> 3) * (FA_BM * 128) + (((i & 7) ^ sw) << 4)) = v;
          }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
      }
      // ---- epilogue: O / l -> bf16 -> staged through shared memory (the P buffer) -> coalesced rows of `out`
      if (ok && n_kv > 0) {
        ok = mbar_wait(o_done, (n_kv - 1) & 1, cta_abort, status, ERR_WAIT_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        constexpr int CH = D / 8;  // 16-byte chunks per output row
        uint8_t* orow = sP + row * (D * 2);
#pragma unroll
        for (int c4 = 0; c4 < D / 32; ++c4) {
          uint32_t r[32];
          if (n_kv > 0) {
            tmem_ld_32x32(lane_addr + 2 * FA_BN + c4 * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * i]) * inv, __uint_as_float(r[8 * i + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
            const int ch = c4 * 4 + i;
            *reinterpret_cast<uint4*>(orow + ((ch ^ (row & (CH - 1))) << 4)) = v;
          }
        }
        if (qi < q_len && lse != nullptr)
          lse[static_cast<size_t>(h) * lse_stride + q_off + qi] = (m_run + log2f(fmaxf(l_run, 1e-38f))) * 0.6931471805599453f;
        fa_named_barrier(1, 128);
        const int t = threadIdx.x - 64;  // 0..127
        const int rows_valid = min(FA_BM, q_len - q0);
        for (int idx = t; idx < rows_valid * CH; idx += 128) {
          const int rr = idx / CH, ch = idx % CH;
          const uint4 v = *reinterpret_cast<const uint4*>(sP + rr * (D * 2) + ((ch ^ (rr & (CH - 1))) << 4));
          *reinterpret_cast<uint4*>(out + static_cast<size_t>(q_off + q0 + rr) * out_stride + h * D + ch * 8) = v;
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);  // let copies in flight land
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, S::TMEM_COLS);
}

template <int D>
static int launch_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* seg, int nseg,
                            int max_q_tiles, int Tq, int Tk, int Hq, int Hkv, int q_stride, int k_stride, int v_stride,
                            int out_stride, int lse_stride, float scale, int* status, cudaStream_t s) {
  using S = FaSmem<D>;
  const CUtensorMap tq = make_tmap_2d(q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tq, size_t(Hq) * D, size_t(q_stride) * 2, FA_BM, 64,
                                      CU_TENSOR_MAP_SWIZZLE_128B);
  const CUtensorMap tk = make_tmap_2d(k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tk, size_t(Hkv) * D, size_t(k_stride) * 2, FA_BN, 64,
                                      CU_TENSOR_MAP_SWIZZLE_128B);
  const CUtensorMap tv = make_tmap_2d(v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tk, size_t(Hkv) * D, size_t(v_stride) * 2, FA_BN, 64,
                                      CU_TENSOR_MAP_SWIZZLE_128B);
  auto kern = flash_fwd_kernel<D>;
  if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), S::TOTAL); e != cudaSuccess) return (int)e;
  return (int)launch_pdl(kern, dim3(max_q_tiles, Hq), dim3(FA_THREADS), S::TOTAL, s, tq, tk, tv,
                         reinterpret_cast<__nv_bfloat16*>(out), lse, seg, nseg, Hq, Hkv, out_stride, lse_stride, scale, status);
}

}  // namespace sb

// q: [Tq, Hq, D] bf16 with row pitch q_stride (elements; the head dim is contiguous), k / v: [Tk, Hkv, D] with pitches
// k_stride / v_stride; out: [Tq, Hq * D] with pitch out_stride; lse: [Hq, lse_stride] fp32 or null. seg: device table of
// nseg x 4 ints (see the top of this file). max_q_tiles: an upper bound of the total number of 128-row query tiles over
// all segments (CTAs beyond the real count exit at once). Base pointers 16-byte aligned, pitches multiples of 8.
// Returns 0, a cudaError_t value, or -1 when the head dim is not 64 or 128.
extern "C" int sb_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* seg, int nseg,
                            int max_q_tiles, int Tq, int Tk, int Hq, int Hkv, int D, int q_stride, int k_stride, int v_stride,
                            int out_stride, int lse_stride, float scale, int* status, cudaStream_t s) {
  if (nseg <= 0 || max_q_tiles <= 0 || Tq <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0) return (int)cudaErrorInvalidValue;
  try {
    if (D == 64)
      return sb::launch_flash_fwd<64>(q, k, v, out, lse, seg, nseg, max_q_tiles, Tq, Tk, Hq, Hkv, q_stride, k_stride, v_stride,
                                      out_stride, lse_stride, scale, status, s);
    if (D == 128)
      return sb::launch_flash_fwd<128>(q, k, v, out, lse, seg, nseg, max_q_tiles, Tq, Tk, Hq, Hkv, q_stride, k_stride,
                                       v_stride, out_stride, lse_stride, scale, status, s);
  } catch (const std::exception& e) {
    sb::set_last_error(e.what());
    return (int)cudaErrorInvalidValue;
  }
  return -1;
}
