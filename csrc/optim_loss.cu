// Optimizer and loss kernels for sm_100a.
//   * sq-norm of a flat gradient buffer (two-stage, deterministic)
//   * fused Adam(W) on fp32 master / m / v shards with unscale + clip + bf16 write-back
//   * vocab(-parallel) softmax statistics over fp32 logits rows: max, sum-exp, target logit,
//     sum p*z  ->  log-prob and entropy; and the matching dlogits kernel
//   * GRPO / PPO-clip / CISPO per-token surrogate with its derivative wrt log-prob
#include "common.cuh"

namespace sb {

// ------------------------------------------------------------------ grad norm
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(256) sqnorm_partial_kernel(const T* __restrict__ g, size_t n, float* __restrict__ partial) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float v = to_f<T>(g[i]);
    s += v * v;
  }
  s = block_sum<256>(s, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

// out[0] (+)= sum(partial)   (single CTA: fixed summation order)
__global__ void __launch_bounds__(256) sum_partials_kernel(const float* __restrict__ partial, int n, float* __restrict__ out,
                                                           int accumulate) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = block_sum<256>(s, scratch);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}

// ----------------------------------------------------------------------- Adam
// ctl[0] = total grad sq-norm (after reduction over all shards/ranks), ctl[1] = skip flag (non-zero: no update).
// clip coefficient = min(1, max_norm / (sqrt(ctl[0]) * grad_scale + 1e-6)) computed on device -> no host sync.
struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale, max_norm;
};

template <typename G>
__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, const G* __restrict__ g,
            __nv_bfloat16* __restrict__ p_bf16, size_t n, AdamArgs a, const float* __restrict__ ctl, int stateless) {
  if (ctl != nullptr && ctl[1] != 0.f) return;
  float coef = a.grad_scale;
  if (ctl != nullptr && a.max_norm > 0.f) {
    const float norm = sqrtf(ctl[0]) * a.grad_scale;
    coef *= fminf(1.f, a.max_norm / (norm + 1e-6f));
  }
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float grad = to_f<G>(g[i]) * coef;
    float pi = p[i];
    float mi, vi;
    if (stateless) {  // moments restart at zero every step
      mi = (1.f - a.beta1) * grad;
      vi = (1.f - a.beta2) * grad * grad;
    } else {
      mi = a.beta1 * m[i] + (1.f - a.beta1) * grad;
      vi = a.beta2 * v[i] + (1.f - a.beta2) * grad * grad;
      m[i] = mi;
      v[i] = vi;
    }
    pi -= a.lr * a.weight_decay * pi;
    pi -= a.lr * (mi / a.bc1) / (sqrtf(vi / a.bc2) + a.eps);
    p[i] = pi;
    if (p_bf16 != nullptr) p_bf16[i] = __float2bfloat16(pi);
  }
}

// --------------------------------------------------- softmax statistics per row
// logits: [T, Vp] fp32 (local vocab shard, global ids [v_lo, v_lo+Vp)). Per row writes
//   stats[t] = {max, sumexp (relative to max), target logit (0 if not owned), sum exp(z-max)*z}
// With tp > 1 the four vectors are combined across ranks by the caller (max: MAX; the
// others after rescaling to the global max: SUM); finalize_logprob_kernel does the
// rescale given the global max.
constexpr int LSE_THREADS = 512;

__global__ void __launch_bounds__(LSE_THREADS)
softmax_stats_kernel(const float* __restrict__ logits, const int* __restrict__ targets, float4* __restrict__ stats, int Vp,
                     size_t ld, int v_lo, float inv_temperature) {
  __shared__ float scratch[32];
  const size_t t = blockIdx.x;
  const float* row = logits + t * ld;
  float mx = -INFINITY, se = 0.f, sz = 0.f;
  const int nvec = Vp >> 2;
  const float4* row4 = reinterpret_cast<const float4*>(row);
  for (int c = threadIdx.x; c < nvec; c += LSE_THREADS) {
    const float4 q = row4[c];
    const float z[4] = {q.x * inv_temperature, q.y * inv_temperature, q.z * inv_temperature, q.w * inv_temperature};
    const float cm = fmaxf(fmaxf(z[0], z[1]), fmaxf(z[2], z[3]));
    if (cm > mx) {
      const float r = __expf(mx - cm);
      se *= r;
      sz *= r;
      mx = cm;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float e = __expf(z[i] - mx);
      se += e;
      sz += e * z[i];
    }
  }
  for (int c = (nvec << 2) + threadIdx.x; c < Vp; c += LSE_THREADS) {
    const float z = row[c] * inv_temperature;
    if (z > mx) {
      const float r = __expf(mx - z);
      se *= r;
      sz *= r;
      mx = z;
    }
    const float e = __expf(z - mx);
    se += e;
    sz += e * z;
  }
  const float gmx = block_max<LSE_THREADS>(mx, scratch);
  const float r = (mx == -INFINITY) ? 0.f : __expf(mx - gmx);
  const float gse = block_sum<LSE_THREADS>(se * r, scratch);
  const float gsz = block_sum<LSE_THREADS>(sz * r, scratch);
  if (threadIdx.x == 0) {
    const int tg = targets[t] - v_lo;
    const float tz = (tg >= 0 && tg < Vp) ? row[tg] * inv_temperature : 0.f;
    stats[t] = make_float4(gmx, gse, tz, gsz);
  }
}

// logp = tz - (log(se) + mx) ; entropy = (log(se)+mx) - sz/se ; lse saved for backward
__global__ void finalize_logprob_kernel(const float4* __restrict__ stats, float* __restrict__ logp,
                                        float* __restrict__ entropy, float* __restrict__ lse, int T) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float4 s = stats[t];
  const float l = logf(s.y) + s.x;
  logp[t] = s.z - l;
  if (entropy != nullptr) entropy[t] = l - s.w / s.y;
  lse[t] = l;
}

// dlogits[t, v] = inv_T * ( g_lp[t] * (1[v==target] - p) - g_ent[t] * p * (log p + H[t]) ),  p = exp(z - lse)
// written as bf16 (feeds the dgrad / wgrad GEMMs).
__global__ void __launch_bounds__(LSE_THREADS)
dlogits_kernel(const float* __restrict__ logits, const int* __restrict__ targets, const float* __restrict__ lse,
               const float* __restrict__ entropy, const float* __restrict__ g_lp, const float* __restrict__ g_ent,
               __nv_bfloat16* __restrict__ dlogits, int Vp, size_t ld, size_t ld_out, int v_lo, float inv_temperature) {
  const size_t t = blockIdx.x;
  const float* row = logits + t * ld;
  __nv_bfloat16* out = dlogits + t * ld_out;
  const float l = lse[t], glp = g_lp[t];
  const float ge = g_ent != nullptr ? g_ent[t] : 0.f;
  const float H = entropy != nullptr ? entropy[t] : 0.f;
  const int tg = targets[t] - v_lo;
  const int nvec = Vp >> 2;
  const float4* row4 = reinterpret_cast<const float4*>(row);
  for (int c = threadIdx.x; c < nvec; c += LSE_THREADS) {
    const float4 q = row4[c];
    const float z[4] = {q.x * inv_temperature, q.y * inv_temperature, q.z * inv_temperature, q.w * inv_temperature};
    float d[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float lp = z[i] - l;
      const float p = __expf(lp);
      float gz = -glp * p;
      if (ge != 0.f) gz -= ge * p * (lp + H);
      if (4 * c + i == tg) gz += glp;
      d[i] = gz * inv_temperature;
    }
    uint2 o;
    o.x = pack_bf16x2(d[0], d[1]);
    o.y = pack_bf16x2(d[2], d[3]);
    *reinterpret_cast<uint2*>(out + 4 * c) = o;
  }
  for (int c = (nvec << 2) + threadIdx.x; c < Vp; c += LSE_THREADS) {
    const float z = row[c] * inv_temperature;
    const float lp = z - l;
    const float p = __expf(lp);
    float gz = -glp * p;
    if (ge != 0.f) gz -= ge * p * (lp + H);
    if (c == tg) gz += glp;
    out[c] = __float2bfloat16(gz * inv_temperature);
  }
}

// ------------------------------------------------------- policy-gradient surrogate
// mode 0: PPO/GRPO clip (optional dual clip eps_c > 1), mode 1: CISPO.
// Inputs per token: logp (new), old_logp, adv, w (loss weight: mask / normaliser).
// Outputs: g_lp[t] = d(sum_t w_t L_t)/d logp_t, and acc[0..3] += {sum w L, sum w clipfrac, sum w (old-new), sum w}
__global__ void __launch_bounds__(256)
pg_loss_kernel(const float* __restrict__ logp, const float* __restrict__ old_logp, const float* __restrict__ adv,
               const float* __restrict__ w, const float* __restrict__ tis, float* __restrict__ g_lp,
               float* __restrict__ per_token_loss, float* __restrict__ acc, int T, float eps_lo, float eps_hi, float eps_c,
               int mode) {
  __shared__ float scratch[32];
  float s_loss = 0.f, s_clip = 0.f, s_kl = 0.f, s_w = 0.f;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x) {
    const float kl = old_logp[t] - logp[t];
    const float ratio = __expf(-kl);
    const float A = adv[t];
    const float wt = w[t] * (tis != nullptr ? tis[t] : 1.f);
    float L, dL, clipped;
    const float rc = fminf(fmaxf(ratio, 1.f - eps_lo), 1.f + eps_hi);
    if (mode == 1) {
      L = -rc * A * logp[t];
      dL = -rc * A;
      clipped = (rc != ratio) ? 1.f : 0.f;
    } else {
      const float l1 = -ratio * A, l2 = -rc * A;
      clipped = (l2 > l1) ? 1.f : 0.f;
      L = fmaxf(l1, l2);
      // derivative wrt logp: d ratio / d logp = ratio ; the clipped branch is flat where rc != ratio
      dL = (l2 > l1) ? ((rc == ratio) ? -ratio * A : 0.f) : -ratio * A;
      if (eps_c > 1.f && A < 0.f) {
        const float l3 = -eps_c * A;
        if (l3 < L) {
          L = l3;
          dL = 0.f;
        }
      }
    }
    if (per_token_loss != nullptr) per_token_loss[t] = L;
    g_lp[t] = dL * wt;
    s_loss += L * wt;
    s_clip += clipped * w[t];
    s_kl += kl * w[t];
    s_w += w[t];
  }
  s_loss = block_sum<256>(s_loss, scratch);
  s_clip = block_sum<256>(s_clip, scratch);
  s_kl = block_sum<256>(s_kl, scratch);
  s_w = block_sum<256>(s_w, scratch);
  if (threadIdx.x == 0) {
    atomicAdd(acc + 0, s_loss);
    atomicAdd(acc + 1, s_clip);
    atomicAdd(acc + 2, s_kl);
    atomicAdd(acc + 3, s_w);
  }
}

}  // namespace sb

extern "C" int sb_sqnorm(const void* g, long n, int is_bf16, float* partial, int num_partials, float* out, int accumulate,
                         cudaStream_t s) {
  if (is_bf16)
    sb::sqnorm_partial_kernel<__nv_bfloat16><<<num_partials, 256, 0, s>>>((const __nv_bfloat16*)g, (size_t)n, partial);
  else
    sb::sqnorm_partial_kernel<float><<<num_partials, 256, 0, s>>>((const float*)g, (size_t)n, partial);
  sb::sum_partials_kernel<<<1, 256, 0, s>>>(partial, num_partials, out, accumulate);
  return (int)cudaGetLastError();
}

extern "C" int sb_adam(float* p, float* m, float* v, const void* g, int g_is_bf16, void* p_bf16, long n, float lr,
                       float beta1, float beta2, float eps, float wd, float bc1, float bc2, float grad_scale,
                       float max_norm, const float* ctl, int stateless, cudaStream_t s) {
  if (n == 0) return 0;
  sb::AdamArgs a{lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, max_norm};
  size_t blocks = ((size_t)n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (g_is_bf16)
    sb::adam_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, s>>>(p, m, v, (const __nv_bfloat16*)g, (__nv_bfloat16*)p_bf16,
                                                              (size_t)n, a, ctl, stateless);
  else
    sb::adam_kernel<float><<<(int)blocks, 256, 0, s>>>(p, m, v, (const float*)g, (__nv_bfloat16*)p_bf16, (size_t)n, a, ctl,
                                                      stateless);
  return (int)cudaGetLastError();
}

extern "C" int sb_softmax_stats(const float* logits, const int* targets, float* stats, int T, int Vp, long ld, int v_lo,
                                float inv_temperature, cudaStream_t s) {
  if (T == 0) return 0;
  if ((ld % 4) != 0 || (reinterpret_cast<uintptr_t>(logits) & 15) != 0) return (int)cudaErrorInvalidValue;
  sb::softmax_stats_kernel<<<T, sb::LSE_THREADS, 0, s>>>(logits, targets, reinterpret_cast<float4*>(stats), Vp, (size_t)ld,
                                                        v_lo, inv_temperature);
  return (int)cudaGetLastError();
}

extern "C" int sb_finalize_logprob(const float* stats, float* logp, float* entropy, float* lse, int T, cudaStream_t s) {
  if (T == 0) return 0;
  sb::finalize_logprob_kernel<<<(T + 255) / 256, 256, 0, s>>>(reinterpret_cast<const float4*>(stats), logp, entropy, lse, T);
  return (int)cudaGetLastError();
}

extern "C" int sb_dlogits(const float* logits, const int* targets, const float* lse, const float* entropy,
                          const float* g_lp, const float* g_ent, void* dlogits, int T, int Vp, long ld, long ld_out,
                          int v_lo, float inv_temperature, cudaStream_t s) {
  if (T == 0) return 0;
  if ((ld % 4) != 0 || (ld_out % 4) != 0) return (int)cudaErrorInvalidValue;
  sb::dlogits_kernel<<<T, sb::LSE_THREADS, 0, s>>>(logits, targets, lse, entropy, g_lp, g_ent, (__nv_bfloat16*)dlogits, Vp,
                                                  (size_t)ld, (size_t)ld_out, v_lo, inv_temperature);
  return (int)cudaGetLastError();
}

extern "C" int sb_pg_loss(const float* logp, const float* old_logp, const float* adv, const float* w, const float* tis,
                          float* g_lp, float* per_token_loss, float* acc, int T, float eps_lo, float eps_hi, float eps_c,
                          int mode, cudaStream_t s) {
  if (T == 0) return 0;
  int blocks = (T + 255) / 256;
  if (blocks > 148) blocks = 148;
  sb::pg_loss_kernel<<<blocks, 256, 0, s>>>(logp, old_logp, adv, w, tis, g_lp, per_token_loss, acc, T, eps_lo, eps_hi,
                                           eps_c, mode);
  return (int)cudaGetLastError();
}
