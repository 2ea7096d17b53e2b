// Token sampling for the rollout engine (sm_100a): temperature, top-k, top-p (nucleus),
// min-p, Gumbel-max draw with a counter-based Philox stream keyed by the request's
// seed, log-prob of the sampled token (renormalised over the kept set when the
// nucleus is active) and optional emission of the kept-id set for top-p replay.
//
// One CTA per request row. Without top-k/top-p the kernel is a single pass over the
// logits row (online softmax + perturbed arg-max). With a nucleus, the exact cut-off
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

  // ---- pass 1: online max / sum-exp, and (unfiltered) the Gumbel-perturbed arg-max
  float mx = -INFINITY, se = 0.f;
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int base = threadIdx.x * 4; base < V; base += SAMPLE_THREADS * 4) {
    uint32_t rnd[4] = {0, 0, 0, 0};
    if (!greedy && !filtered) philox4(seed, pos, static_cast<uint32_t>(base >> 2), rnd);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = base + i;
      if (c < V) {
        const float z = to_float(row[c]) * inv_t;
        if (z > mx) {
          se *= __expf(mx - z);
          mx = z;
        }
        se += __expf(z - mx);
        if (!filtered) {
          const float score = greedy ? z : z + gumbel_from_bits(rnd[i]);
          best = argmax_combine(best, ArgMax{score, c});
        }
      }
    }
  }
  const float gmx = block_max<SAMPLE_THREADS>(mx, scratch);
  const float gse = block_sum<SAMPLE_THREADS>(mx == -INFINITY ? 0.f : se * __expf(mx - gmx), scratch);
  const float lse = __logf(gse) + gmx;

  if (!filtered) {
    const ArgMax w = block_argmax(best, am);
    if (threadIdx.x == 0) {
      token[b] = w.i;
      logprob[b] = to_float(row[w.i]) * inv_t - lse;  // greedy: inv_t == 1, log-prob under the unscaled distribution
      if (kept_count != nullptr) {
        kept_count[b] = greedy ? 1 : 0;  // 0 = "whole vocabulary kept"
        if (greedy && kept_ids != nullptr && kept_cap > 0) kept_ids[static_cast<size_t>(b) * kept_cap] = w.i;
      }
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
