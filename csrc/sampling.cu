// Token sampling for the rollout engine (sm_100a): temperature, top-k, top-p (nucleus),
// min-p, Gumbel-max draw with a counter-based Philox stream keyed by the request's
// seed, log-prob of the sampled token (renormalised over the kept set when the
// nucleus is active) and optional emission of the kept-id set for top-p replay.
//
// One CTA per request row. Without top-k/top-p the kernel is a single vectorised pass over the
// logits row (online softmax) followed by a two-stage inverse-CDF draw that uses two uniforms per
// row and re-reads only one thread's share of the row. With a nucleus, the exact cut-off
// probability is found by a 4-level radix select over the fp32 bit pattern of p
// (histograms of mass and count per 8-bit digit), then one more pass draws the token.
#include "common.cuh"

namespace sb {

constexpr int SAMPLE_THREADS = 512;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

// 4 x 32 random bits for (seed, stream position, index)
__device__ __forceinline__ void philox4(uint64_t seed, uint32_t pos, uint32_t idx, uint32_t (&out)[4]) {
  uint32_t c[4] = {idx, pos, 0x9E3779B9u, 0u};
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}

__device__ __forceinline__ float gumbel_from_bits(uint32_t bits) {
  const float u = (static_cast<float>(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0,1)
  return -__logf(-__logf(u));
}

struct ArgMax {
  float v;
  int i;
};

__device__ __forceinline__ ArgMax argmax_combine(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ __forceinline__ ArgMax block_argmax(ArgMax x, ArgMax* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = argmax_combine(x, y);
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[wid] = x;
  __syncthreads();
  if (wid == 0) {
    ArgMax y = (lane < SAMPLE_THREADS / 32) ? sh[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax z;
      z.v = __shfl_xor_sync(0xffffffffu, y.v, o);
      z.i = __shfl_xor_sync(0xffffffffu, y.i, o);
      y = argmax_combine(y, z);
    }
    if (lane == 0) sh[0] = y;
  }
  __syncthreads();
  return sh[0];
}

// Inclusive prefix sum over the block in thread order. `sh` holds >= 32 floats; all threads must call.
__device__ __forceinline__ float block_scan_incl(float v, float* sh) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  __syncthreads();
  if (lane == 31) sh[wid] = v;
  __syncthreads();
  if (wid == 0) {
    float w = lane < SAMPLE_THREADS / 32 ? sh[lane] : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    sh[lane] = w;
  }
  __syncthreads();
  return v + (wid > 0 ? sh[wid - 1] : 0.f);
}

__device__ __forceinline__ int block_min_int(int v, int* sh) {
  v = __reduce_min_sync(0xffffffffu, v);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[wid] = v;
  __syncthreads();
  int r = lane < SAMPLE_THREADS / 32 ? sh[lane] : 0x7fffffff;
  return __reduce_min_sync(0xffffffffu, r);
}

// logits [B, V] (fp32 or bf16). Per row parameters in arrays of length B.
//   temperature (>0; <=0 means greedy), top_k (<=0: off), top_p (>=1: off), min_p (<=0: off)
//   seeds[b], positions[b] (decode step index of the request: advances the random stream)
// Outputs: token[b], logprob[b]; kept ids (optional): kept_ids[b * kept_cap + j], kept_count[b].
template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const T* __restrict__ logits, size_t ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const uint64_t* __restrict__ seeds, const int* __restrict__ positions, int* __restrict__ token,
              float* __restrict__ logprob, int* __restrict__ kept_ids, int* __restrict__ kept_count, int kept_cap) {
  __shared__ float scratch[32];
  __shared__ ArgMax am[32];
  __shared__ float h_mass[256];
  __shared__ int h_cnt[256];
  __shared__ uint32_t s_prefix;
  __shared__ float s_mass_above;
  __shared__ int s_cnt_above;
  __shared__ int s_kept;
  __shared__ float scan_sh[33];
  __shared__ int red_i[32];

  pdl_wait();  // inputs come from the previous kernel in the stream
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const T* row = logits + static_cast<size_t>(b) * ld;
  const float temp = temperature[b];
  const bool greedy = temp <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temp;
  const int k = top_k != nullptr ? top_k[b] : 0;
  const float tp = top_p != nullptr ? top_p[b] : 1.f;
  const float mp = min_p != nullptr ? min_p[b] : 0.f;
  const bool filtered = !greedy && ((k > 0 && k < V) || tp < 1.f || mp > 0.f);
  const uint64_t seed = seeds != nullptr ? seeds[b] : 0x1234ull + b;
  const uint32_t pos = positions != nullptr ? static_cast<uint32_t>(positions[b]) : 0u;

  // Four consecutive logits (scaled by 1/T) starting at `base` (a multiple of 4): one vector load when the row
  // is aligned for it, scalar loads with -inf past the end otherwise.
  const bool vec_ok = (ld % 4 == 0) && (reinterpret_cast<uintptr_t>(logits) % (4 * sizeof(T)) == 0);
  auto load4 = [&](int base, float (&z)[4]) {
    if (vec_ok && base + 4 <= V) {
      if constexpr (sizeof(T) == 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + base);
        z[0] = v.x; z[1] = v.y; z[2] = v.z; z[3] = v.w;
      } else {
        const uint2 v = *reinterpret_cast<const uint2*>(row + base);
        z[0] = __uint_as_float(v.x << 16); z[1] = __uint_as_float(v.x & 0xffff0000u);
        z[2] = __uint_as_float(v.y << 16); z[3] = __uint_as_float(v.y & 0xffff0000u);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) z[i] *= inv_t;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) z[i] = (base + i < V) ? to_float(row[base + i]) * inv_t : -INFINITY;
    }
  };

  // ---- pass 1: online max / sum-exp per thread (one rescale per group of four), greedy arg-max on the way
  float mx = -INFINITY, se = 0.f;
  ArgMax best{-INFINITY, 0x7fffffff};
  constexpr int UNROLL = 4;  // groups whose loads are issued together, so each thread keeps 64 bytes in flight
  for (int base0 = threadIdx.x * 4; base0 < V; base0 += SAMPLE_THREADS * 4 * UNROLL) {
    float z[UNROLL][4];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int base = base0 + u * SAMPLE_THREADS * 4;
      if (base < V) {
        load4(base, z[u]);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) z[u][i] = -INFINITY;
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int base = base0 + u * SAMPLE_THREADS * 4;
      const float m4 = fmaxf(fmaxf(z[u][0], z[u][1]), fmaxf(z[u][2], z[u][3]));
      if (m4 == -INFINITY) continue;  // fully masked (or past the end)
      if (m4 > mx) {
        se *= __expf(mx - m4);
        mx = m4;
      }
      se += (__expf(z[u][0] - mx) + __expf(z[u][1] - mx)) + (__expf(z[u][2] - mx) + __expf(z[u][3] - mx));
      if (greedy) {
#pragma unroll
        for (int i = 0; i < 4; ++i) best = argmax_combine(best, ArgMax{z[u][i], base + i});
      }
    }
  }
  const float gmx = block_max<SAMPLE_THREADS>(mx, scratch);
  const float my_mass = mx == -INFINITY ? 0.f : se * __expf(mx - gmx);  // this thread's share, relative to exp(gmx)
  const float gse = block_sum<SAMPLE_THREADS>(my_mass, scratch);
  const float lse = __logf(gse) + gmx;

  if (greedy) {
    const ArgMax w = block_argmax(best, am);
    if (threadIdx.x == 0) {
      token[b] = w.i;
      logprob[b] = to_float(row[w.i]) - lse;  // inv_t == 1: log-prob under the unscaled distribution
      if (kept_count != nullptr) {
        kept_count[b] = 1;
        if (kept_ids != nullptr && kept_cap > 0) kept_ids[static_cast<size_t>(b) * kept_cap] = w.i;
      }
    }
    return;
  }

  if (!filtered) {
    // ---- two-stage inverse-CDF draw with two uniforms per row: first the thread whose share of the mass contains
    //      u1 * total, then, inside that thread's strided set of groups, the group and element containing u2 * share.
    //      Only the chosen thread's groups (V / 2048 of them) are read again.
    uint32_t rnd[4];
    philox4(seed, pos, 0u, rnd);
    const float u1 = (static_cast<float>(rnd[0] >> 8) + 0.5f) * (1.0f / 16777216.0f);
    const float u2 = (static_cast<float>(rnd[1] >> 8) + 0.5f) * (1.0f / 16777216.0f);
    const float incl = block_scan_incl(my_mass, scan_sh);
    // first thread whose inclusive sum reaches the target; rounding can leave none: then the last thread with mass
    const float target = u1 * gse;
    int cand = (my_mass > 0.f && incl >= target) ? static_cast<int>(threadIdx.x) : 0x7fffffff;
    int last = my_mass > 0.f ? static_cast<int>(threadIdx.x) : -1;
    cand = block_min_int(cand, red_i);
    last = -block_min_int(-last, red_i);
    const int owner = max(cand != 0x7fffffff ? cand : last, 0);
    // stage 2: thread j handles group j of the owner's set (element base = owner * 4 + j * THREADS * 4)
    float carry = 0.f;  // mass of the groups before this round of SAMPLE_THREADS groups
    int found = 0x7fffffff;
    float found_excl = 0.f;
    int last_group = -1;
    const int ngroups = (V - owner * 4 + SAMPLE_THREADS * 4 - 1) / (SAMPLE_THREADS * 4);
    // share of the owner, recomputed relative to exp(gmx) in the same order the scan below adds it up
    float share = 0.f;
    for (int j0 = 0; j0 < ngroups; j0 += SAMPLE_THREADS) {
      const int j = j0 + threadIdx.x;
      float z[4], c = 0.f;
      if (j < ngroups) {
        load4(owner * 4 + j * SAMPLE_THREADS * 4, z);
#pragma unroll
        for (int i = 0; i < 4; ++i) c += __expf(z[i] - gmx);
      }
      share += block_sum<SAMPLE_THREADS>(c, scratch);
    }
    const float target2 = u2 * share;
    for (int j0 = 0; j0 < ngroups && found == 0x7fffffff; j0 += SAMPLE_THREADS) {
      const int j = j0 + threadIdx.x;
      float z[4], c = 0.f;
      if (j < ngroups) {
        load4(owner * 4 + j * SAMPLE_THREADS * 4, z);
#pragma unroll
        for (int i = 0; i < 4; ++i) c += __expf(z[i] - gmx);
      }
      const float inc2 = carry + block_scan_incl(c, scan_sh);
      const int hit = (c > 0.f && inc2 >= target2) ? j : 0x7fffffff;
      const int lg = c > 0.f ? j : -1;
      found = block_min_int(hit, red_i);
      last_group = max(last_group, -block_min_int(-lg, red_i));
      if (found == j) scan_sh[32] = inc2 - c;  // exclusive sum at the chosen group
      __syncthreads();
      if (found != 0x7fffffff) found_excl = scan_sh[32];
      carry += block_sum<SAMPLE_THREADS>(c, scratch);
    }
    if (threadIdx.x == 0) {
      const bool exact = found != 0x7fffffff;
      const int g = exact ? found : last_group;
      const int base = owner * 4 + g * SAMPLE_THREADS * 4;
      float z[4];
      load4(base, z);
      int pick = -1, last_ok = 0;
      float run = exact ? found_excl : 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float e = __expf(z[i] - gmx);
        if (e > 0.f) last_ok = i;
        run += e;
        if (pick < 0 && exact && e > 0.f && run >= target2) pick = i;
      }
      if (pick < 0) pick = last_ok;
      token[b] = base + pick;
      logprob[b] = z[pick] - lse;
      if (kept_count != nullptr) kept_count[b] = 0;  // 0 = "whole vocabulary kept"
    }
    return;
  }

  // ---- radix select of the cut-off: smallest probability bit pattern `thr` such that the mass of
  // tokens with p > thr ... i.e. keep token i iff mass(p_j > p_i) <= top_p and count(p_j > p_i) < top_k.
  if (threadIdx.x == 0) {
    s_prefix = 0;
    s_mass_above = 0.f;
    s_cnt_above = 0;
  }
  const float p_max = __expf(gmx - lse);
  for (int level = 3; level >= 0; --level) {
    for (int i = threadIdx.x; i < 256; i += SAMPLE_THREADS) {
      h_mass[i] = 0.f;
      h_cnt[i] = 0;
    }
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const int shift = level * 8;
    const uint32_t hi_mask = level == 3 ? 0u : (0xffffffffu << (shift + 8));
    for (int c = threadIdx.x; c < V; c += SAMPLE_THREADS) {
      const float p = __expf(to_float(row[c]) * inv_t - lse);
      const uint32_t bits = __float_as_uint(p);
      if ((bits & hi_mask) == (prefix & hi_mask)) {
        const int d = (bits >> shift) & 0xff;
        atomicAdd(&h_mass[d], p);
        atomicAdd(&h_cnt[d], 1);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float mass = s_mass_above;
      int cnt = s_cnt_above;
      int d = 255;
      // walk digits from the largest probability down; stop in the digit where a limit is crossed
      for (; d > 0; --d) {
        const float nm = mass + h_mass[d];
        const int nc = cnt + h_cnt[d];
        if (h_cnt[d] > 0 && (nm > tp || (k > 0 && nc >= k))) break;
        mass = nm;
        cnt = nc;
      }
      s_prefix = prefix | (static_cast<uint32_t>(d) << shift);
      s_mass_above = mass;
      s_cnt_above = cnt;
    }
    __syncthreads();
  }
  // tokens with bits > s_prefix are all kept; tokens equal to the pivot pattern are kept too (the
  // pivot is the token at which the limit is crossed: mass strictly above it is still <= top_p).
  const uint32_t thr_bits = s_prefix;
  const float minp_thr = mp > 0.f ? p_max * mp : 0.f;
  if (threadIdx.x == 0) s_kept = 0;
  __syncthreads();

  // ---- final pass: kept mass, Gumbel-max among kept tokens, optional id emission
  float kept_mass = 0.f;
  best = ArgMax{-INFINITY, 0x7fffffff};
  for (int base = threadIdx.x * 4; base < V; base += SAMPLE_THREADS * 4) {
    uint32_t rnd[4];
    philox4(seed, pos, static_cast<uint32_t>(base >> 2), rnd);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = base + i;
      if (c < V) {
        const float z = to_float(row[c]) * inv_t;
        const float p = __expf(z - lse);
        if (__float_as_uint(p) >= thr_bits && p >= minp_thr) {
          kept_mass += p;
          best = argmax_combine(best, ArgMax{z + gumbel_from_bits(rnd[i]), c});
          if (kept_ids != nullptr) {
            const int slot = atomicAdd(&s_kept, 1);
            if (slot < kept_cap) kept_ids[static_cast<size_t>(b) * kept_cap + slot] = c;
          }
        }
      }
    }
  }
  kept_mass = block_sum<SAMPLE_THREADS>(kept_mass, scratch);
  const ArgMax w = block_argmax(best, am);
  if (threadIdx.x == 0) {
    token[b] = w.i;
    logprob[b] = to_float(row[w.i]) * inv_t - lse - __logf(kept_mass);
    if (kept_count != nullptr) kept_count[b] = kept_ids != nullptr ? min(s_kept, kept_cap) : -1;
  }
}

}  // namespace sb

extern "C" int sb_sample(const void* logits, int is_bf16, long ld, int B, int V, const float* temperature,
                         const int* top_k, const float* top_p, const float* min_p, const unsigned long long* seeds,
                         const int* positions, int* token, float* logprob, int* kept_ids, int* kept_count, int kept_cap,
                         cudaStream_t s) {
  if (B == 0) return 0;
  if (is_bf16)
    return (int)sb::launch_pdl(sb::sample_kernel<__nv_bfloat16>, dim3(B), dim3(sb::SAMPLE_THREADS), 0, s,
                               (const __nv_bfloat16*)logits, (size_t)ld, V, temperature, top_k, top_p, min_p,
                               (const uint64_t*)seeds, positions, token, logprob, kept_ids, kept_count, kept_cap);
  return (int)sb::launch_pdl(sb::sample_kernel<float>, dim3(B), dim3(sb::SAMPLE_THREADS), 0, s, (const float*)logits, (size_t)ld,
                             V, temperature, top_k, top_p, min_p, (const uint64_t*)seeds, positions, token, logprob, kept_ids,
                             kept_count, kept_cap);
}
