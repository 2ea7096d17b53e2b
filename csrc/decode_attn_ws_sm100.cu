// Paged decode attention for head dim 64, warp-specialised and persistent (sm_100a).
//
// Same math as decode_attn_sm100.cu (S^T = K·Q^T and O^T = V^T·P^T on tcgen05, one token per thread for the softmax),
// reorganised so that an SM keeps FOUR softmax chains in flight instead of two and no softmax thread ever issues a
// copy or an MMA:
//
//   warps 0, 2      TMA producers: warp 0 brings Q of every work item (ring of 6 slots) and K tiles (128 tokens, ring of
//                   5), warp 2 brings V tiles (ring of 7); lane p fetches page p of a tile
//   warps 1, 3      MMA issuers (lane 0 each; one thread cannot issue fast enough for four groups): warp 1 issues S^T(t)
//                   as soon as K(t) has landed and the owning group has drained its previous S^T (this frees the K
//                   slot); warp 3 issues O^T(t) as soon as that tile's P^T is ready (this frees the V slot)
//   warps 4..19     four softmax groups of 128 threads; tile t belongs to group t mod 4, which reads S^T from TMEM,
//                   forms p = 2^(s - max), writes P^T (bf16) to shared memory and folds the previous tile's O^T into
//                   registers. Each group keeps its own running (max, sum, accumulator): it is a split of the
//                   sequence, and writes an un-normalised partial result per work item.
//   combine kernel  merges the 4 x splits partials of every (request, head).
//
// A CTA walks work items (request, kv head, split) blockIdx.x, blockIdx.x + gridDim.x, ...; tiles are numbered through
// all its items, so the pipeline never drains between items. Every wait is an mbarrier wait with a 2 s bound (also the
// exchange inside a softmax group): on expiry the CTA records a status word, every role leaves its loop, copies in
// flight are given time to land, TMEM is freed and the kernel returns.
#include "common.cuh"

namespace sb {

// K and V tiles live in separate rings: a K slot is free again as soon as S^T of its tile has been computed, a V slot
// only after the tile's softmax and O^T product, so V gets the deeper ring and each is loaded by its own warp.
constexpr int WS_TILE = 128, WS_D = 64, WS_NWG = 4, WS_NK = 5, WS_NV = 7, WS_NQ = 6, WS_MAXG = 8;
constexpr int WS_THREADS = 128 + 128 * WS_NWG;  // K producer, S^T issuer, V producer, O^T issuer, 4 softmax groups
constexpr int WS_KV_TILE = WS_TILE * 128;        // one K (or V) tile: 128 tokens x 128 bytes
constexpr int WS_P_BYTES = 2 * WS_MAXG * 128;    // P^T: 2 chunks of 64 tokens x 8 heads x 128 B
constexpr int WS_Q_BYTES = 16 * 128;             // 16 rows (heads) x 64 dims
constexpr int WS_NBAR = 2 * WS_NK + 2 * WS_NV + 6 * WS_NWG + 2 * WS_NQ;
constexpr int WS_SMEM = (WS_NK + WS_NV) * WS_KV_TILE + WS_NWG * WS_P_BYTES + WS_NQ * WS_Q_BYTES + WS_NBAR * 8 + 64 + 1024;

__device__ __forceinline__ float ws_warp_max(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float ws_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

struct WsItem {
  int b, kvh, sp, t_begin, t_end, ntiles;
};

// Sequence length of work item `it` (0 past the end). Every role loads the length of the NEXT item while it works on the
// current one, so this global load is never on anybody's critical path.
__device__ __forceinline__ int ws_len(int it, int num_items, int Hkv, int splits, const int* __restrict__ seq_lens) {
  return it < num_items ? __ldg(seq_lens + it / (splits * Hkv)) : 0;
}

// Work item `it` -> request, kv head, split and its token range (the same arithmetic in every role).
__device__ __forceinline__ WsItem ws_item(int it, int Hkv, int splits, int len) {
  WsItem w;
  w.sp = it % splits;
  w.kvh = (it / splits) % Hkv;
  w.b = it / (splits * Hkv);
  const int tiles_total = (len + WS_TILE - 1) / WS_TILE;
  const int per = (tiles_total + splits - 1) / splits;
  w.t_begin = min(len, w.sp * per * WS_TILE);
  w.t_end = min(len, (w.sp + 1) * per * WS_TILE);
  w.ntiles = w.t_end > w.t_begin ? (w.t_end - w.t_begin + WS_TILE - 1) / WS_TILE : 0;
  return w;
}

template <int G>
__global__ void __launch_bounds__(WS_THREADS, 1)
decode_attn_ws_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      const __grid_constant__ CUtensorMap tmQ, const int* __restrict__ block_table,
                      const int* __restrict__ seq_lens, float* __restrict__ part_o, float* __restrict__ part_ml, int num_items,
                      int Hq, int Hkv, int page_size, int page_shift, int max_pages, int splits, float scale, int* status) {
  static_assert(G <= WS_MAXG, "this kernel keeps 8 query heads per kv head at most");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + WS_NK * WS_KV_TILE;
  uint8_t* sP = sV + WS_NV * WS_KV_TILE;
  uint8_t* sQ = sP + WS_NWG * WS_P_BYTES;
  uint64_t* full_k = reinterpret_cast<uint64_t*>(sQ + WS_NQ * WS_Q_BYTES);
  uint64_t* k_empty = full_k + WS_NK;
  uint64_t* full_v = k_empty + WS_NK;
  uint64_t* v_empty = full_v + WS_NV;
  uint64_t* s_full = v_empty + WS_NV;
  uint64_t* s_free = s_full + WS_NWG;
  uint64_t* p_ready = s_free + WS_NWG;
  uint64_t* o_full = p_ready + WS_NWG;
  uint64_t* o_free = o_full + WS_NWG;
  uint64_t* wg_bar = o_free + WS_NWG;
  uint64_t* q_full = wg_bar + WS_NWG;
  uint64_t* q_empty = q_full + WS_NQ;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_empty + WS_NQ);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ __align__(16) float red_m[WS_NWG][2][WS_MAXG][4];  // [group][parity][head][warp]
  __shared__ float red_l[WS_NWG][4][WS_MAXG];
  constexpr int BT_CACHE = 256, BT_PER_LANE = BT_CACHE / 32;
  __shared__ int bt_s[2][2][BT_CACHE];  // [K or V producer][item parity][page]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float scale_log2 = scale * 1.4426950408889634f;

  if (tid == 0) {
    for (int s = 0; s < WS_NK; ++s) {
      mbar_init(&full_k[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < WS_NV; ++s) {
      mbar_init(&full_v[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int w = 0; w < WS_NWG; ++w) {
      mbar_init(&s_full[w], 1);
      mbar_init(&s_free[w], 4);
      mbar_init(&p_ready[w], 4);
      mbar_init(&o_full[w], 1);
      mbar_init(&o_free[w], 4);
      mbar_init(&wg_bar[w], 4);
    }
    for (int s = 0; s < WS_NQ; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    *cta_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmQ);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 64 * WS_NWG);  // per group: S^T at +0, O^T at +32 (16 columns used of each 32)
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();

  // ------------------------------------------------------------------------------------------ TMA producers
  // Run by warp 0 for K (and Q) and by warp 2 for V. Block-table entries are staged in shared memory one item ahead
  // (lane l keeps entries l, l + 32, ... of the NEXT item in registers while the current item's tiles are issued, and
  // stores them afterwards), sequence lengths two items ahead: no global load sits between two tile issues.
  auto produce = [&](const bool is_k) {
    const int ring = is_k ? WS_NK : WS_NV;
    uint64_t* full = is_k ? full_k : full_v;
    uint64_t* emp = is_k ? k_empty : v_empty;
    uint8_t* base = is_k ? sK : sV;
    const CUtensorMap* map = is_k ? &tmK : &tmV;
    int (*bt_mine)[BT_CACHE] = bt_s[is_k ? 0 : 1];
    int gt = 0, iq = -1;  // iq counts the items that have tiles: only those use a Q slot
    bool ok = true;
    auto bt_fetch = [&](const WsItem& x, int (&regs)[BT_PER_LANE]) {
      const int* row = block_table + static_cast<size_t>(x.b) * max_pages + (x.t_begin >> page_shift);
      const int n = x.ntiles > 0 ? min(BT_CACHE, ((x.t_end - x.t_begin + page_size - 1) >> page_shift)) : 0;
#pragma unroll
      for (int j = 0; j < BT_PER_LANE; ++j) regs[j] = lane + 32 * j < n ? __ldg(row + lane + 32 * j) : 0;
    };
    auto bt_store = [&](int buf, const int (&regs)[BT_PER_LANE]) {
#pragma unroll
      for (int j = 0; j < BT_PER_LANE; ++j) bt_mine[buf][lane + 32 * j] = regs[j];
      __syncwarp();
    };
    int it = blockIdx.x;
    int len_cur = ws_len(it, num_items, Hkv, splits, seq_lens);
    int len_next = ws_len(it + gridDim.x, num_items, Hkv, splits, seq_lens);
    int regs[BT_PER_LANE];
    if (it < num_items) {
      bt_fetch(ws_item(it, Hkv, splits, len_cur), regs);
      bt_store(0, regs);
    }
    for (int k = 0; it < num_items && ok; it += gridDim.x, ++k) {
      const WsItem w = ws_item(it, Hkv, splits, len_cur);
      const int it_n = it + gridDim.x;
      const WsItem wn = ws_item(it_n < num_items ? it_n : it, Hkv, splits, it_n < num_items ? len_next : 0);
      const int len_after = ws_len(it_n + gridDim.x, num_items, Hkv, splits, seq_lens);  // consumed two items from now
      if (it_n < num_items) bt_fetch(wn, regs);                                          // consumed one item from now
      const int* bt_cur = bt_mine[k & 1];
      if (w.ntiles > 0) {
        ++iq;
        if (is_k) {
          const int qs = iq % WS_NQ;
          if (lane == 0) {
            ok = mbar_wait(&q_empty[qs], ((iq / WS_NQ) & 1) ^ 1, cta_abort, status, ERR_WAIT_EMPTY);
            if (ok) {
              mbar_arrive_expect_tx(&q_full[qs], WS_Q_BYTES);
              tma_load_3d(sQ + qs * WS_Q_BYTES, &tmQ, &q_full[qs], 0, w.kvh * G, w.b);
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
        }
        const int* bt_row = block_table + static_cast<size_t>(w.b) * max_pages + (w.t_begin >> page_shift);
        for (int i = 0; i < w.ntiles && ok; ++i, ++gt) {
          const int s = gt % ring;
          const int valid = min(WS_TILE, w.t_end - (w.t_begin + i * WS_TILE));
          const int npages = (valid + page_size - 1) >> page_shift;
          const int pi = ((i * WS_TILE) >> page_shift) + lane;  // page index within the item's range
          int slot0 = 0;
          if (lane < npages) slot0 = (pi < BT_CACHE ? bt_cur[pi] : __ldg(bt_row + pi)) * page_size;
          if (lane == 0) {
            ok = mbar_wait(&emp[s], ((gt / ring) & 1) ^ 1, cta_abort, status, ERR_WAIT_EMPTY);
            if (ok) mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(npages * page_size * 128));
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (ok && lane < npages)
            tma_load_3d(base + s * WS_KV_TILE + lane * page_size * 128, map, &full[s], 0, w.kvh, slot0);
          __syncwarp();
        }
      }
      if (it_n < num_items) bt_store((k + 1) & 1, regs);
      len_cur = len_next;
      len_next = len_after;
    }
  };

  if (warp == 0) {
    produce(true);
  } else if (warp == 2) {
    produce(false);
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------------------ S^T issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(WS_TILE, 16, 1, 1, 0, 0);  // A = K tile (K-major), B = Q (K-major)
      bool ok = true;
      int gt = 0, iq = -1;
      int len_cur = ws_len(blockIdx.x, num_items, Hkv, splits, seq_lens);
      for (int it = blockIdx.x; it < num_items && ok; it += gridDim.x) {
        const WsItem wi = ws_item(it, Hkv, splits, len_cur);
        len_cur = ws_len(it + gridDim.x, num_items, Hkv, splits, seq_lens);  // for the next item; lands during this one
        if (wi.ntiles == 0) continue;
        ++iq;
        const int qs = iq % WS_NQ;
        ok = mbar_wait(&q_full[qs], (iq / WS_NQ) & 1, cta_abort, status, ERR_WAIT_FULL);
        for (int i = 0; i < wi.ntiles && ok; ++i, ++gt) {
          const int w = gt % WS_NWG, n = gt / WS_NWG, s = gt % WS_NK;
          if (!mbar_wait(&full_k[s], (gt / WS_NK) & 1, cta_abort, status, ERR_WAIT_FULL) ||
              !mbar_wait(&s_free[w], (n & 1) ^ 1, cta_abort, status, ERR_WAIT_TMEM_EMPTY)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t k_addr = smem_u32(sK + s * WS_KV_TILE);
          const uint32_t q_addr = smem_u32(sQ + qs * WS_Q_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_base + w * 64, make_smem_desc(k_addr + k * 32, 16, 1024, UMMA_SWIZZLE_128B),
                     make_smem_desc(q_addr + k * 32, 16, 1024, UMMA_SWIZZLE_128B), idesc_s, k != 0 ? 1u : 0u);
          umma_commit(&s_full[w]);
          umma_commit(&k_empty[s]);  // the K slot is free once S^T exists
          if (i == wi.ntiles - 1) umma_commit(&q_empty[qs]);  // the item's last use of its Q slot
        }
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------------------------------------ O^T issuer
    if (lane == 0) {
      constexpr uint32_t idesc_o = make_idesc(128, 16, 1, 1, 1, 0);  // A = V tile read MN-major, B = P^T
      bool ok = true;
      auto issue_o = [&](int gt) -> bool {
        const int w = gt % WS_NWG, n = gt / WS_NWG, s = gt % WS_NV;
        if (!mbar_wait(&p_ready[w], n & 1, cta_abort, status, ERR_WAIT_FULL) ||
            !mbar_wait(&full_v[s], (gt / WS_NV) & 1, cta_abort, status, ERR_WAIT_FULL) ||
            !mbar_wait(&o_free[w], (n & 1) ^ 1, cta_abort, status, ERR_WAIT_TMEM_EMPTY))
          return false;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + s * WS_KV_TILE);
        const uint32_t p_addr = smem_u32(sP + w * WS_P_BYTES);
        // V^T as the A operand (M = 128 rows: the head dim and, above it, 64 rows of whatever follows the V slot in
        // shared memory; those product rows are never read). 64-token chunks kc, 16-token K steps k inside a chunk.
#pragma unroll
        for (int kc = 0; kc < 2; ++kc)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_base + w * 64 + 32, make_smem_desc(v_addr + (kc * 4 + k) * 2048, WS_TILE * 128, 1024, UMMA_SWIZZLE_128B),
                     make_smem_desc(p_addr + kc * (WS_MAXG * 128) + k * 32, 16, 1024, UMMA_SWIZZLE_128B), idesc_o,
                     (kc | k) != 0 ? 1u : 0u);
        umma_commit(&o_full[w]);
        umma_commit(&v_empty[s]);
        return true;
      };
      int gt = 0;
      int len_cur = ws_len(blockIdx.x, num_items, Hkv, splits, seq_lens);
      for (int it = blockIdx.x; it < num_items && ok; it += gridDim.x) {
        const WsItem wi = ws_item(it, Hkv, splits, len_cur);
        len_cur = ws_len(it + gridDim.x, num_items, Hkv, splits, seq_lens);
        for (int i = 0; i < wi.ntiles && ok; ++i, ++gt) ok = issue_o(gt);
      }
    }
  } else {
    // --------------------------------------------------------------------------------------- softmax groups
    const int w = (warp - 4) >> 2;   // group
    const int q = warp & 3;          // TMEM lane quarter this warp may touch
    const int wt = q * 32 + lane;    // token of the tile, and (below 64) output dim, owned by this thread
    const uint32_t t_s = tmem_base + w * 64 + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t t_o = t_s + 32;
    const bool merges = wt < WS_D;   // warp-uniform
    uint32_t xph = 0;                // phase of the group's exchange barrier
    // exchange inside the group: every warp's lane 0 arrives after its shared-memory writes, everybody waits
    auto group_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(&wg_bar[w]);
      const bool r = mbar_wait(&wg_bar[w], xph & 1, cta_abort, status, ERR_WAIT_PEER);
      ++xph;
      return __all_sync(0xffffffffu, r);
    };
    int gt = 0;
    bool ok = true;
    int len_cur = ws_len(blockIdx.x, num_items, Hkv, splits, seq_lens);
    for (int it = blockIdx.x; it < num_items && ok; it += gridDim.x) {
      const WsItem wi = ws_item(it, Hkv, splits, len_cur);
      len_cur = ws_len(it + gridDim.x, num_items, Hkv, splits, seq_lens);  // for the next item; lands during this one
      float acc[G], m_run[G], l_thr[G], keep_prev[G], gain_prev[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        acc[g] = 0.f;
        m_run[g] = -INFINITY;
        l_thr[g] = 0.f;
        keep_prev[g] = 1.f;
        gain_prev[g] = 0.f;
      }
      // own tiles of this item: global numbers gt + i with (gt + i) % NWG == w
      const int first = (w - gt % WS_NWG + WS_NWG) % WS_NWG;
      const int mine = first < wi.ntiles ? (wi.ntiles - first + WS_NWG - 1) / WS_NWG : 0;
      auto merge = [&](int n) -> bool {  // fold the O^T of own tile number n (of this group) into the accumulator
        bool r = mbar_wait(&o_full[w], n & 1, cta_abort, status, ERR_WAIT_TMEM_FULL);
        r = __all_sync(0xffffffffu, r);
        if (!r) return false;
        tc_fence_after();
        if (merges) {
          uint32_t o[32];
          tmem_ld_32x32(t_o, o);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < G; ++g) acc[g] = acc[g] * keep_prev[g] + __uint_as_float(o[g]) * gain_prev[g];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_free[w]);
        return true;
      };
      for (int j = 0; j < mine && ok; ++j) {
        const int g_t = gt + first + j * WS_NWG;  // global tile number
        const int n = g_t / WS_NWG, s = g_t % WS_NV, par = n & 1;
        const int t0 = wi.t_begin + (first + j * WS_NWG) * WS_TILE;
        const int valid = min(WS_TILE, wi.t_end - t0);
        // ---- scores of this thread's token for the G heads
        ok = mbar_wait(&s_full[w], par, cta_abort, status, ERR_WAIT_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float sc[G];
        {
          uint32_t r[32];
          tmem_ld_32x32(t_s, r);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_free[w]);  // S^T is in registers: the next product may overwrite it
#pragma unroll
          for (int g = 0; g < G; ++g) sc[g] = (wt < valid) ? __uint_as_float(r[g]) * scale_log2 : -INFINITY;
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float wm = ws_warp_max(sc[g]);
          if (lane == 0) red_m[w][par][g][q] = wm;
        }
        ok = group_sync();
        if (!ok) break;
        // ---- the previous own tile's product is long done: fold it in (this also frees P^T and O^T of the group)
        if (j > 0) {
          ok = merge(n - 1);
          if (!ok) break;
        }
        // ---- p = 2^(s - tile max), running max / sum bookkeeping, P^T to shared memory
        const int kc = wt >> 6, col = wt & 63;
        uint8_t* p_col = sP + w * WS_P_BYTES + kc * (WS_MAXG * 128) + (col & 7) * 2;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float4 wmx = *reinterpret_cast<const float4*>(red_m[w][par][g]);
          const float mt = fmaxf(fmaxf(wmx.x, wmx.y), fmaxf(wmx.z, wmx.w));
          const float p = ws_exp2(sc[g] - mt);
          const float nm = fmaxf(m_run[g], mt);
          const float keep = ws_exp2(m_run[g] - nm);
          const float gain = ws_exp2(mt - nm);
          l_thr[g] = l_thr[g] * keep + p * gain;
          m_run[g] = nm;
          keep_prev[g] = keep;
          gain_prev[g] = gain;
          *reinterpret_cast<__nv_bfloat16*>(p_col + g * 128 + (((col >> 3) ^ (g & 7)) << 4)) = __float2bfloat16(p);
        }
        if (valid < WS_TILE) {
          // rows past the end of the sequence hold whatever an older tile left there: p is 0 for them, but 0 x NaN
          // would poison O^T, so they are cleared once the copy of this tile's V has landed
          ok = mbar_wait(&full_v[s], (g_t / WS_NV) & 1, cta_abort, status, ERR_WAIT_FULL);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (wt >= valid) {
            uint4* vrow = reinterpret_cast<uint4*>(sV + s * WS_KV_TILE + wt * 128);
#pragma unroll
            for (int c = 0; c < 8; ++c) vrow[c] = make_uint4(0, 0, 0, 0);
          }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[w]);
        if (j == mine - 1) ok = merge(n);  // last own tile of the item: wait for its product right away
      }
      if (!ok) break;
      // ---- partial result of this group for the item (an empty marker if it had no tile)
      float l_tot[G];
#pragma unroll
      for (int g = 0; g < G; ++g) l_tot[g] = 0.f;
      if (mine > 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float ws = warp_sum(l_thr[g]);
          if (lane == 0) red_l[w][q][g] = ws;
        }
        ok = group_sync();
        if (!ok) break;
#pragma unroll
        for (int g = 0; g < G; ++g) l_tot[g] = (red_l[w][0][g] + red_l[w][1][g]) + (red_l[w][2][g] + red_l[w][3][g]);
        ok = group_sync();  // red_l is read before the next item may overwrite it
        if (!ok) break;
      }
      const int nsplit = splits * WS_NWG;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int h = wi.kvh * G + g;
        const size_t base = (static_cast<size_t>(wi.b) * Hq + h) * nsplit + wi.sp * WS_NWG + w;
        if (mine > 0 && merges) part_o[base * WS_D + wt] = acc[g];
        if (wt == 0) {
          part_ml[base * 2 + 0] = mine > 0 ? m_run[g] * 0.6931471805599453f : -INFINITY;  // natural-log domain
          part_ml[base * 2 + 1] = mine > 0 ? l_tot[g] : 0.f;
        }
      }
      gt += wi.ntiles;
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    const unsigned long long t_a = globaltimer_ns();
    while (globaltimer_ns() - t_a < 200000ull) __nanosleep(1000);  // copies still in flight may land
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, 64 * WS_NWG);
}

// q viewed as [B, Hq, 64] with a token pitch of q_stride elements; box = 16 heads x 64 dims of one request (heads past
// Hq read as zero: they only feed S^T columns nobody looks at).
static CUtensorMap ws_make_q_tmap(const void* q, int B, int Hq, int q_stride) {
  CUtensorMap m;
  cuuint64_t dims[3] = {(cuuint64_t)WS_D, (cuuint64_t)Hq, (cuuint64_t)B};
  cuuint64_t strides[2] = {(cuuint64_t)WS_D * 2, (cuuint64_t)q_stride * 2};
  cuuint32_t box[3] = {64, 16, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = get_encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled (q) failed: " + std::to_string(int(r)));
  return m;
}

// Cache viewed as [num_slots, Hkv, 64] with arbitrary (16-byte multiple) slot and head pitches, in elements: the
// slot-major layout [slots, Hkv, D] has (Hkv * D, D), the head-major one [Hkv, slots, D] has (D, slots * D).
static CUtensorMap ws_make_cache_tmap(const void* base, int num_slots, int Hkv, int page_size, long slot_stride,
                                      long head_stride) {
  CUtensorMap m;
  cuuint64_t dims[3] = {(cuuint64_t)WS_D, (cuuint64_t)Hkv, (cuuint64_t)num_slots};
  cuuint64_t strides[2] = {(cuuint64_t)head_stride * 2, (cuuint64_t)slot_stride * 2};
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
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled (kv cache) failed: " + std::to_string(int(r)));
  return m;
}

// out[b, h, :] from the nsplit partials of one (request, head): sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M).
__global__ void decode_attn_ws_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              __nv_bfloat16* __restrict__ out, int nsplit, int out_stride, int Hq) {
  pdl_wait();
  pdl_launch_dependents();
  const int bh = blockIdx.x, b = bh / Hq, h = bh % Hq, d = threadIdx.x;
  const float* ml = part_ml + static_cast<size_t>(bh) * nsplit * 2;
  float gm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) gm = fmaxf(gm, ml[2 * s]);
  float gl = 0.f, o = 0.f;
  for (int s = 0; s < nsplit; ++s)
    if (ml[2 * s] != -INFINITY) {
      const float e = __expf(ml[2 * s] - gm);
      gl += ml[2 * s + 1] * e;
      o += part_o[(static_cast<size_t>(bh) * nsplit + s) * WS_D + d] * e;
    }
  out[static_cast<size_t>(b) * out_stride + static_cast<size_t>(h) * WS_D + d] = __float2bfloat16(gl > 0.f ? o / gl : 0.f);
}

template <int G>
static int ws_launch(int grid, cudaStream_t s, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tq, const int* bt,
                     const int* sl, float* po, float* pml, int num_items, int Hq, int Hkv, int page_size, int page_shift,
                     int max_pages, int splits, float scale, int* status) {
  auto kern = decode_attn_ws_kernel<G>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WS_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)launch_pdl(kern, dim3(grid), dim3(WS_THREADS), WS_SMEM, s, tk, tv, tq, bt, sl, po, pml, num_items, Hq, Hkv, page_size,
                         page_shift, max_pages, splits, scale, status);
}

}  // namespace sb

// Head dim 64, at most 8 query heads per kv head. part_o / part_ml: workspaces [B, Hq, 4 * splits, 64] and
// [B, Hq, 4 * splits, 2] fp32 (always used). Returns 0, a cudaError_t value, or -1 for shapes this kernel does not cover.
extern "C" int sb_paged_decode_ws(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                  const int* seq_lens, void* out, float* part_o, float* part_ml, int B, int Hq, int Hkv, int D,
                                  int page_size, int max_pages, int num_slots, int q_stride, int out_stride, int splits,
                                  float scale, int* status, int num_sms, long kv_slot_stride, long kv_head_stride,
                                  cudaStream_t s) {
  if (B == 0) return 0;
  if ((kv_slot_stride & 7) || (kv_head_stride & 7)) return -1;
  if (D != sb::WS_D || Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > sb::WS_MAXG || splits < 1) return -1;
  const int G = Hq / Hkv;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  if ((1 << page_shift) != page_size || page_size < 16 || page_size > 128) return -1;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (q_stride & 7) || (reinterpret_cast<uintptr_t>(out) & 1) ||
      (reinterpret_cast<uintptr_t>(k_cache) & 127) || (reinterpret_cast<uintptr_t>(v_cache) & 127))
    return -1;
  try {
    const CUtensorMap tk = sb::ws_make_cache_tmap(k_cache, num_slots, Hkv, page_size, kv_slot_stride, kv_head_stride);
    const CUtensorMap tv = sb::ws_make_cache_tmap(v_cache, num_slots, Hkv, page_size, kv_slot_stride, kv_head_stride);
    const CUtensorMap tq = sb::ws_make_q_tmap(q, B, Hq, q_stride);
    const int num_items = B * Hkv * splits;
    const int grid = num_items < num_sms ? num_items : num_sms;
    int rc = -1;
#define SB_WS(GV)                                                                                                         \
  if (G == GV)                                                                                                             \
    rc = sb::ws_launch<GV>(grid, s, tk, tv, tq, block_table, seq_lens, part_o, part_ml, num_items, Hq, Hkv, page_size, page_shift, \
                           max_pages, splits, scale, status);
    SB_WS(1) SB_WS(2) SB_WS(3) SB_WS(4) SB_WS(5) SB_WS(6) SB_WS(7) SB_WS(8)
#undef SB_WS
    if (rc != 0) return rc;
    return (int)sb::launch_pdl(sb::decode_attn_ws_combine_kernel, dim3(B * Hq), dim3(sb::WS_D), 0, s, (const float*)part_o,
                               (const float*)part_ml, (__nv_bfloat16*)out, splits * sb::WS_NWG, out_stride, Hq);
  } catch (const std::exception& e) {
    sb::set_last_error(e.what());
    return (int)cudaErrorInvalidValue;
  }
}
