// Paged decode attention for head dim 64, warp-specialised and persistent (sm_100a).
//
// Same math as decode_attn_sm100.cu (S^T = K·Q^T and O^T = V^T·P^T on tcgen05, one token per thread for the softmax),
// reorganised so that an SM keeps FOUR softmax chains in flight instead of two and no softmax thread ever issues a
// copy or an MMA:
//
//   warp 20         scheduler: walks the CTA's work items (WsSched), reads their block-table entries and publishes one
//                   queue entry per tile (request, kv head, split, group, valid tokens, first / last flags, the cache
//                   slot of each page). The other four role warps only read entries: the instruction path per tile of
//                   a single-threaded role is what bounds this kernel, so the bookkeeping lives in a warp of its own
//   warps 0, 2      TMA producers: warp 0 brings K tiles (128 tokens, ring of 5) and Q when a group starts an item (two
//                   slots per group), warp 2 brings V tiles (ring of 7); lane p fetches page p of a tile
//   warps 1, 3      MMA issuers (lane 0 each; one thread cannot issue fast enough for four groups): warp 1 issues S^T(t)
//                   as soon as K(t) has landed and the owning group has drained its previous S^T (this frees the K
//                   slot) and tells the group which tile it is through a small mailbox; warp 3 issues O^T(t) as soon as
//                   that tile's P^T is ready (this frees the V slot)
//   warps 4..19     four softmax groups of 128 threads. A group owns one work item (request, kv head, split) at a time,
//                   from its first tile to its last: it reads S^T from TMEM, forms p = 2^(s - max), writes P^T (bf16) to
//                   shared memory, folds the previous tile's O^T into registers, and at the end of the item writes the
//                   output row (or, with splits > 1, an un-normalised partial for the combine kernel).
//
// A CTA's work items are blockIdx.x, blockIdx.x + gridDim.x, ...; a group that finishes its item takes the CTA's next
// one. Tiles flow through the rings round-robin over the groups, so the pipeline never drains between items. Every wait
// is an mbarrier wait with a 2 s bound (also the exchange inside a softmax group): on expiry the CTA records a status
// word, every role leaves its loop, copies in flight are given time to land, TMEM is freed and the kernel returns.
#include "common.cuh"

namespace sb {

// K and V tiles live in separate rings: a K slot is free again as soon as S^T of its tile has been computed, a V slot
// only after the tile's softmax and O^T product, so V gets the deeper ring and each is loaded by its own warp.
constexpr int WS_TILE = 128, WS_D = 64, WS_NWG = 4, WS_NK = 5, WS_NV = 7, WS_NQ = 2 * WS_NWG, WS_MAXG = 8;
constexpr int WS_THREADS = 128 + 128 * WS_NWG + 32;  // K producer, S^T issuer, V producer, O^T issuer, 4 softmax groups, scheduler
constexpr int WS_SCHED_WARP = 4 + 4 * WS_NWG;
constexpr int WS_KV_TILE = WS_TILE * 128;        // one K (or V) tile: 128 tokens x 128 bytes
constexpr int WS_P_BYTES = 2 * WS_MAXG * 128;    // P^T: 2 chunks of 64 tokens x 8 heads x 128 B
constexpr int WS_Q_BYTES = 16 * 128;             // 16 rows (heads) x 64 dims
constexpr int WS_SQ = 16;                         // entries of the tile queue (K producer -> V producer and both issuers)
constexpr int WS_NBAR = 2 * WS_NK + 2 * WS_NV + 8 * WS_NWG + 2 * WS_NQ + 2 * WS_SQ;
constexpr int WS_SMEM = (WS_NK + WS_NV) * WS_KV_TILE + WS_NWG * WS_P_BYTES + WS_NQ * WS_Q_BYTES + WS_NBAR * 8 + 64 + 1024;
// flags of a tile-queue / mailbox word (low 8 bits: valid tokens of the tile; bits 12-13: the group)
constexpr int WS_F_FIRST = 1 << 8, WS_F_LAST = 1 << 9, WS_F_DONE = 1 << 10, WS_F_GROUP_SHIFT = 12;

__device__ __forceinline__ float ws_warp_max(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
// 32 lanes x 8 columns TMEM -> registers: a thread's row of S^T or O^T for the (at most 8) query heads.
__device__ __forceinline__ void ws_tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ float ws_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

struct WsItem {
  int b, kvh, sp, t_begin, t_end, ntiles;
};

// Optional measurement build (-DSB_WS_CHAIN_TIMING): one thread of softmax group 0 of every CTA clocks the segments of
// its per-tile chain and adds them up in ws_chain_ticks: [0] wait for the mailbox and S^T, [1] TMEM read + row maxima,
// [2] exchange inside the group, [3] merge of the previous product (wait for O^T + TMEM read), [4] exp / P^T / fences,
// [5] end of item (last merge, sum exchange, output), [6] tiles counted. ws_issue_ticks, by the two MMA issuers:
// S^T issuer [0] queue entry, [1] K tile landed, [2] group drained its S^T, [3] issue; O^T issuer [4] P^T ready,
// [5] V tile landed, [6] group merged its previous O^T, [7] issue.
#ifdef SB_WS_CHAIN_TIMING
__device__ unsigned long long ws_chain_ticks[8];
__device__ unsigned long long ws_issue_ticks[8];
#define WS_ITICK(slot)                 \
  {                                    \
    const long long now_ = clock64();  \
    itick[slot] += now_ - itick_last;  \
    itick_last = now_;                 \
  }
#define WS_TICK(slot)                                   \
  if (timing) {                                         \
    const long long now_ = clock64();                   \
    tick_acc[slot] += now_ - tick_last;                 \
    tick_last = now_;                                   \
  }
#else
#define WS_TICK(slot)
#define WS_ITICK(slot)
#endif

// Sequence length of work item `it` (0 past the end).
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

// Four values kept in registers and indexed at run time (a chain of selects; no local memory).
struct WsQuad {
  int v0, v1, v2, v3;
  __device__ __forceinline__ int get(int w) const {
    int r = v0;
    r = w == 1 ? v1 : r;
    r = w == 2 ? v2 : r;
    r = w == 3 ? v3 : r;
    return r;
  }
  __device__ __forceinline__ void set(int w, int x) {
    v0 = w == 0 ? x : v0;
    v1 = w == 1 ? x : v1;
    v2 = w == 2 ? x : v2;
    v3 = w == 3 ? x : v3;
  }
  __device__ __forceinline__ void fill(int x) { v0 = v1 = v2 = v3 = x; }
};

template <int G>
__global__ void __launch_bounds__(WS_THREADS, 1)
decode_attn_ws_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      const __grid_constant__ CUtensorMap tmQ, const int* __restrict__ block_table,
                      const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                      float* __restrict__ part_ml, int num_items, int Hq, int Hkv, int page_size, int page_shift,
                      int max_pages, int splits, int out_stride, float scale, int* status, int load_path_only) {
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
  uint64_t* info_full = wg_bar + WS_NWG;
  uint64_t* v_landed = info_full + WS_NWG;
  uint64_t* q_full = v_landed + WS_NWG;
  uint64_t* q_empty = q_full + WS_NQ;
  uint64_t* sq_full = q_empty + WS_NQ;
  uint64_t* sq_empty = sq_full + WS_SQ;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sq_empty + WS_SQ);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ __align__(16) float red_m[WS_NWG][2][WS_MAXG][4];  // [group][tile parity][head][warp]
  __shared__ float red_l[WS_NWG][2][4][WS_MAXG];                 // [group][item parity][warp][head]
  __shared__ __align__(16) int4 info_s[WS_NWG][2];               // mailbox S^T issuer -> group: [group][tile parity]
  // tile queue: the K producer walks the schedule and publishes, per tile, {request, kv head | split << 16, valid tokens |
  // flags | group << 12, pages} and the cache slot of each of the tile's pages; the V producer and the issuers read it
  __shared__ __align__(16) int4 sq_hdr[WS_SQ];
  __shared__ int sq_slot[WS_SQ][8];

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
      mbar_init(&info_full[w], 1);
      mbar_init(&v_landed[w], 1);
    }
    for (int s = 0; s < WS_NQ; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    for (int e = 0; e < WS_SQ; ++e) {
      mbar_init(&sq_full[e], 1);
      mbar_init(&sq_empty[e], 4);  // both producers, both issuers
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

  // ------------------------------------------------------------------------------------------ roles
  if (warp == WS_SCHED_WARP) {
    // ---- scheduler. Lanes 8g .. 8g+7 look after softmax group g (its item and how far it is; the same values in all
    // eight lanes), lane 8g+p after page p of the group's next tile. One round hands items to the groups that ran out
    // (the CTA's next items, in group order), then publishes the next tile of every group that has one, in group
    // order: up to four queue entries per round, with the block-table lookups of all of them in flight together.
    const int g = lane >> 3, p = lane & 7;
    const int ppt = WS_TILE >> page_shift;  // pages per tile: 8, 4, 2 or 1
    const unsigned seg_mask = 0xffu << (g * 8);
    int next_it = blockIdx.x, gt = 0;
    int rem = 0, nt = 0, ib = 0, ikvh = 0, isp = 0, tb = 0, te = 0;
    bool ok = true;
    for (;;) {
      // -- items for the groups that have none
      const bool needy = rem == 0;
      const unsigned need4 = __ballot_sync(0xffffffffu, needy && p == 0);  // bits 0, 8, 16, 24
      const int before = __popc(need4 & ((1u << (g * 8)) - 1u));
      const int cand = next_it + before * static_cast<int>(gridDim.x);
      if (needy && cand < num_items) {
        const WsItem x = ws_item(cand, Hkv, splits, ws_len(cand, num_items, Hkv, splits, seq_lens));
        if (x.ntiles > 0) {
          rem = nt = x.ntiles;
          ib = x.b;
          ikvh = x.kvh;
          isp = x.sp;
          tb = x.t_begin;
          te = x.t_end;
        } else if (splits == 1) {  // nobody else looks at an item without tiles: its (empty) result is written here
          __nv_bfloat16* o = out + static_cast<size_t>(x.b) * out_stride + static_cast<size_t>(x.kvh) * G * WS_D;
          for (int i = p; i < G * WS_D; i += 8) o[i] = __float2bfloat16(0.f);
        } else if (p < G) {
          const size_t idx = (static_cast<size_t>(x.b) * Hq + x.kvh * G + p) * splits + x.sp;
          part_ml[idx * 2 + 0] = -INFINITY;
          part_ml[idx * 2 + 1] = 0.f;
        }
      }
      const int handed = min(__popc(need4), max(0, (num_items - next_it + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x)));
      next_it += handed * static_cast<int>(gridDim.x);
      // -- the next tile of every group that has one
      const bool active = rem > 0;
      const unsigned act4 = __ballot_sync(0xffffffffu, active && p == 0);
      if (act4 == 0) {
        if (next_it >= num_items) break;
        continue;  // only items without tiles this round
      }
      const int my_gt = gt + __popc(act4 & ((1u << (g * 8)) - 1u));
      const int e = my_gt & (WS_SQ - 1);
      int slot0 = 0;
      int4 hdr = make_int4(0, 0, 0, 0);
      if (active) {
        const int r = nt - rem;
        const int valid = min(WS_TILE, te - (tb + r * WS_TILE));
        const int npages = (valid + page_size - 1) >> page_shift;
        if (p < npages)
          slot0 = __ldg(block_table + static_cast<size_t>(ib) * max_pages + (tb >> page_shift) + r * ppt + p) * page_size;
        const int flags = (r == 0 ? WS_F_FIRST : 0) | (rem == 1 ? WS_F_LAST : 0) | (g << WS_F_GROUP_SHIFT);
        hdr = make_int4(ib, ikvh | (isp << 16), valid | flags, npages);
        ok = mbar_wait(&sq_empty[e], ((my_gt / WS_SQ) & 1) ^ 1, cta_abort, status, ERR_WAIT_EMPTY);
      }
      if (!__all_sync(0xffffffffu, ok)) break;
      if (active) {
        if (p == 0) sq_hdr[e] = hdr;
        sq_slot[e][p] = slot0;
        __syncwarp(seg_mask);
        if (p == 0) mbar_arrive(&sq_full[e]);
        --rem;
      }
      gt += __popc(act4);
    }
    if (__all_sync(0xffffffffu, ok)) {  // end of the stream
      const int e = gt & (WS_SQ - 1);
      ok = mbar_wait(&sq_empty[e], ((gt / WS_SQ) & 1) ^ 1, cta_abort, status, ERR_WAIT_EMPTY);
      if (__all_sync(0xffffffffu, ok) && lane == 0) {
        sq_hdr[e] = make_int4(0, 0, WS_F_DONE, 0);
        mbar_arrive(&sq_full[e]);
      }
    }
  } else if (warp == 0 || warp == 2) {
    // ---- K producer (warp 0; also brings Q when a group starts an item) and V producer (warp 2): tile by tile from
    // the queue, lane p copies page p
    const bool is_k = warp == 0;
    const int ring = is_k ? WS_NK : WS_NV;
    uint64_t* full = is_k ? full_k : full_v;
    uint64_t* emp = is_k ? k_empty : v_empty;
    uint8_t* base = is_k ? sK : sV;
    const CUtensorMap* map = is_k ? &tmK : &tmV;
    WsQuad oq;  // per group: items started (K producer only)
    oq.fill(0);
    for (int gt = 0, s = 0, lap = 0;; ++gt) {
      const int e = gt & (WS_SQ - 1);
      bool ok = mbar_wait(&sq_full[e], (gt / WS_SQ) & 1, cta_abort, status, ERR_WAIT_FULL);
      if (!__all_sync(0xffffffffu, ok)) break;
      const int4 h = sq_hdr[e];
      const int slot0 = sq_slot[e][lane & 7];
      __syncwarp();
      if (lane == 0) mbar_arrive(&sq_empty[e]);
      if (h.z & WS_F_DONE) break;
      const int npages = h.w, kvh = h.y & 0xffff;
      if (lane == 0) {
        if (is_k && (h.z & WS_F_FIRST)) {
          const int w = (h.z >> WS_F_GROUP_SHIFT) & 3, ordinal = oq.get(w), qs = w * 2 + (ordinal & 1);
          oq.set(w, ordinal + 1);
          ok = mbar_wait(&q_empty[qs], ((ordinal >> 1) & 1) ^ 1, cta_abort, status, ERR_WAIT_EMPTY);
          if (ok) {
            mbar_arrive_expect_tx(&q_full[qs], WS_Q_BYTES);
            tma_load_3d(sQ + qs * WS_Q_BYTES, &tmQ, &q_full[qs], 0, kvh * G, h.x);
          }
        }
        ok = ok && mbar_wait(&emp[s], (lap & 1) ^ 1, cta_abort, status, ERR_WAIT_EMPTY);
        if (ok) mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(npages * page_size * 128));
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < npages) tma_load_3d(base + s * WS_KV_TILE + lane * page_size * 128, map, &full[s], 0, kvh, slot0);
      __syncwarp();
      if (++s == ring) {
        s = 0;
        ++lap;
      }
    }
  } else if (warp == 1) {
    // ---- S^T issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(WS_TILE, 16, 1, 1, 0, 0);  // A = K tile (K-major), B = Q (K-major)
      WsQuad nq, oq;  // per group: tiles issued, items started
      nq.fill(0);
      oq.fill(0);
      bool done = false;
#ifdef SB_WS_CHAIN_TIMING
      long long itick[4] = {0, 0, 0, 0}, itick_last = clock64();
#endif
      for (int gt = 0;; ++gt) {
        const int e = gt & (WS_SQ - 1), s = gt % WS_NK;
        if (!mbar_wait(&sq_full[e], (gt / WS_SQ) & 1, cta_abort, status, ERR_WAIT_FULL)) break;
        WS_ITICK(0)
        const int4 h = sq_hdr[e];
        mbar_arrive(&sq_empty[e]);
        if (h.z & WS_F_DONE) {
          done = true;
          break;
        }
        const int w = (h.z >> WS_F_GROUP_SHIFT) & 3;
        const bool first = (h.z & WS_F_FIRST) != 0, last = (h.z & WS_F_LAST) != 0;
        const int n = nq.get(w);
        const int started = oq.get(w) + (first ? 1 : 0), ordinal = started - 1;
        oq.set(w, started);
        nq.set(w, n + 1);
        const int qs = w * 2 + (ordinal & 1);
        if (!mbar_wait(&full_k[s], (gt / WS_NK) & 1, cta_abort, status, ERR_WAIT_FULL)) break;
        if (first && !mbar_wait(&q_full[qs], (ordinal >> 1) & 1, cta_abort, status, ERR_WAIT_FULL)) break;
        WS_ITICK(1)
        if (load_path_only) {  // measurement mode: hand the slots straight back to the producers
          mbar_arrive(&k_empty[s]);
          if (last) mbar_arrive(&q_empty[qs]);
          continue;
        }
        // the group has drained S^T of its previous tile (and is therefore done with the mailbox slot of the one before)
        if (!mbar_wait(&s_free[w], (n & 1) ^ 1, cta_abort, status, ERR_WAIT_TMEM_EMPTY)) break;
        WS_ITICK(2)
        info_s[w][n & 1] = make_int4(h.x, h.y, h.z, gt);
        mbar_arrive(&info_full[w]);
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * WS_KV_TILE);
        const uint32_t q_addr = smem_u32(sQ + qs * WS_Q_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(tmem_base + w * 64, make_smem_desc(k_addr + k * 32, 16, 1024, UMMA_SWIZZLE_128B),
                   make_smem_desc(q_addr + k * 32, 16, 1024, UMMA_SWIZZLE_128B), idesc_s, k != 0 ? 1u : 0u);
        umma_commit(&s_full[w]);
        umma_commit(&k_empty[s]);             // the K slot is free once S^T exists
        if (last) umma_commit(&q_empty[qs]);  // the item's last use of its Q slot
        WS_ITICK(3)
      }
#ifdef SB_WS_CHAIN_TIMING
      for (int i = 0; i < 4; ++i) atomicAdd(&ws_issue_ticks[i], static_cast<unsigned long long>(itick[i]));
#endif
      if (done && !load_path_only) {
        for (int w = 0; w < WS_NWG; ++w) {  // tell every group that nothing more will come
          const int n = nq.get(w);
          if (!mbar_wait(&s_free[w], (n & 1) ^ 1, cta_abort, status, ERR_WAIT_TMEM_EMPTY)) break;
          info_s[w][n & 1] = make_int4(0, 0, WS_F_DONE, 0);
          mbar_arrive(&info_full[w]);
        }
      }
    }
  } else if (warp == 3) {
    // ---- O^T issuer
    if (lane == 0) {
      constexpr uint32_t idesc_o = make_idesc(128, 16, 1, 1, 1, 0);  // A = V tile read MN-major, B = P^T
      WsQuad nq;
      nq.fill(0);
#ifdef SB_WS_CHAIN_TIMING
      long long itick[4] = {0, 0, 0, 0}, itick_last = clock64();
#endif
      for (int gt = 0;; ++gt) {
        const int e = gt & (WS_SQ - 1), s = gt % WS_NV;
        if (!mbar_wait(&sq_full[e], (gt / WS_SQ) & 1, cta_abort, status, ERR_WAIT_FULL)) break;
        const int flags = sq_hdr[e].z;
        mbar_arrive(&sq_empty[e]);
        if (flags & WS_F_DONE) break;
        const int w = (flags >> WS_F_GROUP_SHIFT) & 3;
        const int n = nq.get(w);
        nq.set(w, n + 1);
        if (load_path_only) {
          if (!mbar_wait(&full_v[s], (gt / WS_NV) & 1, cta_abort, status, ERR_WAIT_FULL)) break;
          mbar_arrive(&v_empty[s]);
          continue;
        }
        if ((flags & 0xff) < WS_TILE) {
          // a tile that ends inside the sequence: its group clears the V rows past the end before it announces P^T, and
          // may only do so once the copy has landed. This thread sees every V tile land, in order, so it can tell; a
          // group that looked at full_v itself could be a whole lap of the ring away from what the parity bit means.
          if (!mbar_wait(&full_v[s], (gt / WS_NV) & 1, cta_abort, status, ERR_WAIT_FULL)) break;
          mbar_arrive(&v_landed[w]);
        }
        if (!mbar_wait(&p_ready[w], n & 1, cta_abort, status, ERR_WAIT_FULL)) break;
        WS_ITICK(0)
        if (!mbar_wait(&full_v[s], (gt / WS_NV) & 1, cta_abort, status, ERR_WAIT_FULL)) break;
        WS_ITICK(1)
        if (!mbar_wait(&o_free[w], (n & 1) ^ 1, cta_abort, status, ERR_WAIT_TMEM_EMPTY)) break;
        WS_ITICK(2)
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
        WS_ITICK(3)
      }
#ifdef SB_WS_CHAIN_TIMING
      for (int i = 0; i < 4; ++i) atomicAdd(&ws_issue_ticks[4 + i], static_cast<unsigned long long>(itick[i]));
#endif
    }
  } else if (!load_path_only) {
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
    float acc[G], m_run[G], l_thr[G], keep_prev[G], gain_prev[G];
#pragma unroll
    for (int g = 0; g < G; ++g) acc[g] = m_run[g] = l_thr[g] = keep_prev[g] = gain_prev[g] = 0.f;
    auto merge = [&](int n) -> bool {  // fold the O^T of the group's tile number n into the accumulator
      bool r = mbar_wait(&o_full[w], n & 1, cta_abort, status, ERR_WAIT_TMEM_FULL);
      r = __all_sync(0xffffffffu, r);
      if (!r) return false;
      tc_fence_after();
      if (merges) {
        uint32_t o[8];
        ws_tmem_ld_32x8(t_o, o);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < G; ++g) acc[g] = acc[g] * keep_prev[g] + __uint_as_float(o[g]) * gain_prev[g];
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&o_free[w]);
      return true;
    };
    int b = 0, kvh = 0, sp = 0, items_done = 0, npartial = 0;
    bool ok = true;
#ifdef SB_WS_CHAIN_TIMING
    const bool timing = w == 0 && q == 0 && lane == 0;
    long long tick_acc[7] = {0, 0, 0, 0, 0, 0, 0}, tick_last = clock64();
#endif
    for (int n = 0; ok; ++n) {  // the group's tiles, in the order the S^T issuer announces them
      const int par = n & 1;
      ok = mbar_wait(&info_full[w], par, cta_abort, status, ERR_WAIT_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int4 inf = info_s[w][par];
      if (inf.z & WS_F_DONE) break;
      const int valid = inf.z & 0xff;
      const bool first = (inf.z & WS_F_FIRST) != 0, last = (inf.z & WS_F_LAST) != 0;
      const int g_t = inf.w, s = g_t % WS_NV;
      if (first) {
        b = inf.x;
        kvh = inf.y & 0xffff;
        sp = inf.y >> 16;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          acc[g] = 0.f;
          m_run[g] = -INFINITY;
          l_thr[g] = 0.f;
          keep_prev[g] = 1.f;
          gain_prev[g] = 0.f;
        }
      }
      // ---- scores of this thread's token for the G heads
      ok = mbar_wait(&s_full[w], par, cta_abort, status, ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      WS_TICK(0)
      tc_fence_after();
      float sc[G];
      {
        uint32_t r[8];
        ws_tmem_ld_32x8(t_s, r);
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
      WS_TICK(1)
      ok = group_sync();
      if (!ok) break;
      WS_TICK(2)
      // ---- the previous tile's product is long done: fold it in (this also frees P^T and O^T of the group)
      if (!first) {
        ok = merge(n - 1);
        if (!ok) break;
      }
      WS_TICK(3)
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
        // would poison O^T, so they are cleared once the copy of this tile's V has landed (the O^T issuer says when)
        ok = mbar_wait(&v_landed[w], npartial & 1, cta_abort, status, ERR_WAIT_FULL);  // from the O^T issuer
        ++npartial;
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
      WS_TICK(4)
#ifdef SB_WS_CHAIN_TIMING
      tick_acc[6] += 1;
#endif
      if (!last) continue;
      // ---- last tile of the item: wait for its product right away, then write the item's result
      ok = merge(n);
      if (!ok) break;
      const int ip = items_done & 1;  // red_l is double-buffered: the exchange of the next item cannot overtake a reader
      ++items_done;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float ws = warp_sum(l_thr[g]);
        if (lane == 0) red_l[w][ip][q][g] = ws;
      }
      ok = group_sync();
      if (!ok) break;
      float l_tot[G];
#pragma unroll
      for (int g = 0; g < G; ++g) l_tot[g] = (red_l[w][ip][0][g] + red_l[w][ip][1][g]) + (red_l[w][ip][2][g] + red_l[w][ip][3][g]);
      if (splits == 1) {
        if (merges) {
          __nv_bfloat16* o = out + static_cast<size_t>(b) * out_stride + static_cast<size_t>(kvh) * G * WS_D + wt;
#pragma unroll
          for (int g = 0; g < G; ++g) o[g * WS_D] = __float2bfloat16(acc[g] / l_tot[g]);
        }
      } else {
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const size_t idx = (static_cast<size_t>(b) * Hq + kvh * G + g) * splits + sp;
          if (merges) part_o[idx * WS_D + wt] = acc[g];
          if (wt == 0) {
            part_ml[idx * 2 + 0] = m_run[g] * 0.6931471805599453f;  // natural-log domain
            part_ml[idx * 2 + 1] = l_tot[g];
          }
        }
      }
      WS_TICK(5)
    }
#ifdef SB_WS_CHAIN_TIMING
    if (timing)
      for (int i = 0; i < 7; ++i) atomicAdd(&ws_chain_ticks[i], static_cast<unsigned long long>(tick_acc[i]));
#endif
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
                     const int* sl, __nv_bfloat16* out, float* po, float* pml, int num_items, int Hq, int Hkv, int page_size,
                     int page_shift, int max_pages, int splits, int out_stride, float scale, int* status, int load_path_only) {
  auto kern = decode_attn_ws_kernel<G>;
  if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), WS_SMEM); e != cudaSuccess) return (int)e;
  return (int)launch_pdl(kern, dim3(grid), dim3(WS_THREADS), WS_SMEM, s, tk, tv, tq, bt, sl, out, po, pml, num_items, Hq, Hkv,
                         page_size, page_shift, max_pages, splits, out_stride, scale, status, load_path_only);
}

static int g_ws_load_path_only = 0;

}  // namespace sb

// Measurement switch: with a non-zero value the kernel's producers run as usual and every landed tile is handed straight
// back (no products, no softmax, no output): its duration is what the copy path alone costs for a given batch.
extern "C" void sb_paged_decode_ws_load_path_only(int on) { sb::g_ws_load_path_only = on; }

#ifdef SB_WS_CHAIN_TIMING
// Reads (and with `reset` clears) the counters of a measurement build into out[16]: chain, then issuers.
extern "C" int sb_paged_decode_ws_chain_ticks(unsigned long long* out, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out, sb::ws_chain_ticks, sizeof(unsigned long long) * 8);
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out + 8, sb::ws_issue_ticks, sizeof(unsigned long long) * 8);
  if (e == cudaSuccess && reset) {
    const unsigned long long zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    e = cudaMemcpyToSymbol(sb::ws_chain_ticks, zero, sizeof(zero));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(sb::ws_issue_ticks, zero, sizeof(zero));
  }
  return (int)e;
}
#endif

// Head dim 64, at most 8 query heads per kv head. part_o / part_ml: workspaces [B, Hq, splits, 64] and [B, Hq, splits, 2]
// fp32, used (with the combine kernel) when splits > 1; with one split the kernel writes `out` itself. Returns 0, a cudaError_t value, or -1 for shapes this kernel does not cover.
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
#define SB_WS(GV)                                                                                                        \
  if (G == GV)                                                                                                            \
    rc = sb::ws_launch<GV>(grid, s, tk, tv, tq, block_table, seq_lens, (__nv_bfloat16*)out, part_o, part_ml, num_items, Hq, Hkv, \
                           page_size, page_shift, max_pages, splits, out_stride, scale, status, sb::g_ws_load_path_only);
    SB_WS(1) SB_WS(2) SB_WS(3) SB_WS(4) SB_WS(5) SB_WS(6) SB_WS(7) SB_WS(8)
#undef SB_WS
    if (rc != 0 || splits == 1 || sb::g_ws_load_path_only) return rc;
    return (int)sb::launch_pdl(sb::decode_attn_ws_combine_kernel, dim3(B * Hq), dim3(sb::WS_D), 0, s, (const float*)part_o,
                               (const float*)part_ml, (__nv_bfloat16*)out, splits, out_stride, Hq);
  } catch (const std::exception& e) {
    sb::set_last_error(e.what());
    return (int)cudaErrorInvalidValue;
  }
}
