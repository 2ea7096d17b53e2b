// Data-parallel optimizer step fused with its collectives over NVLink peer memory (ZeRO-1):
//
//   sb_dp_reduce_shard   reduce-scatter: every rank sums ITS shard of the gradient buffer over all ranks, reading the
//                        peers' buffers directly (P2P loads through their symmetric-memory pointers, or one
//                        multimem.ld_reduce through the NVSwitch multicast address, where the switch does the sum),
//                        keeps the sum in its own buffer and produces the partial squared norm in the same pass.
//   sb_dp_adam_bcast     Adam(W) on the shard (fp32 master / moments, clip coefficient from the global norm) and
//                        all-gather: the new bf16 parameters are stored straight into every rank's parameter buffer
//                        (P2P stores, or one multimem.st that the switch replicates).
//   sb_symm_barrier      all ranks meet; signal words live in each rank's symmetric signal pad. The wait is bounded
//                        (sb_set_peer_wait_limit_ns, 2 s unless changed): on expiry the kernel records ERR_WAIT_PEER in
//                        the status word and returns, it never spins forever.
//
// A non-zero status word is sticky until the host clears it. Every kernel here looks at it first: a barrier still
// raises its own flag (so the peers are not held up) but does not wait; the reduce and the Adam kernel touch no data;
// the partial-sum kernel turns it into the "skip this step" flag ctl[1], which the caller all-reduces together with
// the squared norm, so that after one expired wait EVERY rank skips the update and the parameters stay unchanged and
// identical. The host reads the status word where it reads the gradient norm and raises.
//
// Order per step:  barrier -> reduce_shard -> (all-reduce of one scalar: the squared norm) -> adam_bcast -> barrier.
// The gradient traffic is what an NCCL reduce-scatter moves, and the parameter traffic what an all-gather moves, but
// the reduced gradient and the updated parameter never make an extra trip through HBM between collective and math.
// One process per GPU: the kernels of different ranks wait on one another only across GPUs.
#include "common.cuh"

namespace sb {

struct PeerPtrs {
  void* p[8];
};

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// One block, one thread per peer. Slot layout in every rank's pad: words [base + r] = last epoch rank r announced here.
__global__ void symm_barrier_kernel(PeerPtrs pads, int rank, int world, uint32_t epoch, int base, int* status,
                                    unsigned long long limit_ns) {
  const int p = threadIdx.x;
  if (p < world) {
    const bool failed = status != nullptr && *reinterpret_cast<volatile int*>(status) != 0;
    __threadfence_system();  // everything this GPU wrote before the barrier is visible to peers that see the flag
    st_release_sys(static_cast<uint32_t*>(pads.p[p]) + base + rank, epoch);
    if (failed) return;  // an earlier wait expired: announce, do not wait again
    const uint32_t* mine = static_cast<const uint32_t*>(pads.p[rank]) + base + p;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t it = 0;
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++it & 0xff) == 0 && globaltimer_ns() - t0 > limit_ns) {
        if (status) atomicCAS(status, 0, ERR_WAIT_PEER | (p << 8));
        break;
      }
    }
  }
}

// Same barrier with the epoch kept in device memory (`counter`, advanced by the kernel): the launch arguments are
// constant, so the barrier still synchronises when it is replayed from a CUDA graph.
__global__ void symm_barrier_dev_kernel(PeerPtrs pads, int rank, int world, uint32_t* counter, int base, int* status,
                                        unsigned long long limit_ns) {
  const int p = threadIdx.x;
  if (p < world) {
    const bool failed = status != nullptr && *reinterpret_cast<volatile int*>(status) != 0;
    const uint32_t epoch = *counter + 1;
    __syncwarp((1u << world) - 1u);
    if (p == 0) *counter = epoch;
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(pads.p[p]) + base + rank, epoch);
    if (failed) return;
    const uint32_t* mine = static_cast<const uint32_t*>(pads.p[rank]) + base + p;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t it = 0;
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++it & 0xff) == 0 && globaltimer_ns() - t0 > limit_ns) {
        if (status) atomicCAS(status, 0, ERR_WAIT_PEER | (p << 8));
        break;
      }
    }
  }
}

__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}

__device__ __forceinline__ void multimem_st_b32x4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// out[i] = sum_r grads_r[off + i] for i in [0, n) (n % 4 == 0); partials[block] = sum of squares of this block's part.
// MC: grads.p[0] is the multicast address of the buffer (the switch returns the sum over all ranks).
template <bool MC>
__global__ void __launch_bounds__(256)
dp_reduce_shard_kernel(PeerPtrs grads, int world, int rank, size_t off, size_t n, float* __restrict__ out,
                       float* __restrict__ partials, const int* __restrict__ status) {
  __shared__ float scratch[32];
  float ss = 0.f;
  if (status != nullptr && *status != 0) {  // the barrier before this kernel gave up: the peers' buffers may be unfinished
    if (threadIdx.x == 0) partials[blockIdx.x] = 0.f;
    return;
  }
  const size_t nvec = n >> 2;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float4 acc;
    if constexpr (MC) {
      acc = multimem_ld_reduce_f32x4(static_cast<const float*>(grads.p[0]) + off + 4 * i);
    } else {
      acc = make_float4(0.f, 0.f, 0.f, 0.f);
      // start at the own rank and walk the ring so that the N ranks do not all read the same peer at once
      for (int k = 0; k < world; ++k) {
        const int r = (rank + k) % world;
        const float4 g = reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[r]) + off)[i];
        acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
      }
    }
    reinterpret_cast<float4*>(out)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  ss = block_sum<256>(ss, scratch);
  if (threadIdx.x == 0) partials[blockIdx.x] = ss;
}

// ctl[slot] += sum(partials[0..n)) in a fixed order (one block), so the norm does not depend on scheduling.
__global__ void dp_sum_partials_kernel(const float* __restrict__ partials, int n, float* __restrict__ ctl, int slot,
                                       const int* __restrict__ status) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partials[i];
  s = block_sum<256>(s, scratch);
  if (threadIdx.x == 0) {
    ctl[slot] += s;
    if (status != nullptr && *status != 0) ctl[1] += 1.f;  // summed over ranks by the caller: everyone skips the step
  }
}

struct DpAdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale, max_norm;
};

// Adam(W) over the shard (same arithmetic as adam_kernel in optim_loss.cu), then the new bf16 values go to every
// rank's parameter buffer at [off, off + n). n % 8 == 0 so one thread produces one 16-byte store per peer.
template <bool MC>
__global__ void __launch_bounds__(256)
dp_adam_bcast_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, const float* __restrict__ g,
                     PeerPtrs params, int world, int rank, size_t off, size_t n, DpAdamArgs a,
                     const float* __restrict__ ctl, int stateless) {
  // non-finite gradients, or a wait that expired on some rank: the whole step is skipped on every rank
  if (ctl != nullptr && ctl[1] != 0.f) return;
  float coef = a.grad_scale;
  if (ctl != nullptr && a.max_norm > 0.f) {
    const float norm = sqrtf(ctl[0]) * a.grad_scale;
    coef *= fminf(1.f, a.max_norm / (norm + 1e-6f));
  }
  const size_t nvec = n >> 3;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float out[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const size_t j = 2 * i + h;
      const float4 g4 = reinterpret_cast<const float4*>(g)[j];
      float4 p4 = reinterpret_cast<float4*>(p)[j];
      float4 m4 = make_float4(0.f, 0.f, 0.f, 0.f), v4 = m4;
      if (!stateless) {
        m4 = reinterpret_cast<float4*>(m)[j];
        v4 = reinterpret_cast<float4*>(v)[j];
      }
      const float gg[4] = {g4.x * coef, g4.y * coef, g4.z * coef, g4.w * coef};
      float pp[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mi = stateless ? (1.f - a.beta1) * gg[e] : a.beta1 * mm[e] + (1.f - a.beta1) * gg[e];
        const float vi = stateless ? (1.f - a.beta2) * gg[e] * gg[e] : a.beta2 * vv[e] + (1.f - a.beta2) * gg[e] * gg[e];
        mm[e] = mi;
        vv[e] = vi;
        float pi = pp[e];
        pi -= a.lr * a.weight_decay * pi;
        pi -= a.lr * (mi / a.bc1) / (sqrtf(vi / a.bc2) + a.eps);
        pp[e] = pi;
        out[4 * h + e] = pi;
      }
      reinterpret_cast<float4*>(p)[j] = make_float4(pp[0], pp[1], pp[2], pp[3]);
      if (!stateless) {
        reinterpret_cast<float4*>(m)[j] = make_float4(mm[0], mm[1], mm[2], mm[3]);
        reinterpret_cast<float4*>(v)[j] = make_float4(vv[0], vv[1], vv[2], vv[3]);
      }
    }
    uint4 w;
    w.x = pack_bf16x2(out[0], out[1]);
    w.y = pack_bf16x2(out[2], out[3]);
    w.z = pack_bf16x2(out[4], out[5]);
    w.w = pack_bf16x2(out[6], out[7]);
    if constexpr (MC) {
      multimem_st_b32x4(static_cast<__nv_bfloat16*>(params.p[0]) + off + 8 * i, w);
    } else {
      for (int k = 0; k < world; ++k) {
        const int r = (rank + k) % world;
        reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[r]) + off)[i] = w;
      }
    }
  }
}

}  // namespace sb

// Wait limit of every kernel that waits for another GPU, in nanoseconds (0 restores the 2 s default). Process-wide.
extern "C" void sb_set_peer_wait_limit_ns(unsigned long long ns) { sb::peer_wait_limit_ns() = ns ? ns : sb::WAIT_LIMIT_NS; }
extern "C" unsigned long long sb_get_peer_wait_limit_ns(void) { return sb::peer_wait_limit_ns(); }

extern "C" int sb_symm_barrier(const void* const* pads, int rank, int world, unsigned epoch, int base_word, int* status,
                               cudaStream_t s) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return (int)cudaErrorInvalidValue;
  sb::PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = const_cast<void*>(pads[i]);
  sb::symm_barrier_kernel<<<1, 32, 0, s>>>(pp, rank, world, epoch, base_word, status, sb::peer_wait_limit_ns());
  return (int)cudaGetLastError();
}

extern "C" int sb_symm_barrier_dev(const void* const* pads, int rank, int world, unsigned* counter, int base_word,
                                   int* status, cudaStream_t s) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || counter == nullptr) return (int)cudaErrorInvalidValue;
  sb::PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = const_cast<void*>(pads[i]);
  sb::symm_barrier_dev_kernel<<<1, 32, 0, s>>>(pp, rank, world, counter, base_word, status, sb::peer_wait_limit_ns());
  return (int)cudaGetLastError();
}

// grads: `world` pointers to every rank's fp32 gradient buffer (own included), or, with multicast != 0, one multicast
// address in grads[0]. out: where this rank keeps the reduced shard (usually its own buffer at `off`). partials: scratch
// of at least 1184 floats. ctl[0] accumulates the shard's squared norm.
// status: the device status word (may be null); when it is non-zero the kernel reads nothing and ctl[1] is raised.
extern "C" int sb_dp_reduce_shard(const void* const* grads, int world, int rank, int multicast, long off, long n, float* out,
                                  float* partials, float* ctl, const int* status, cudaStream_t s) {
  if (n == 0) return 0;
  if (world < 1 || world > 8 || (n & 3) || (off & 3)) return (int)cudaErrorInvalidValue;
  sb::PeerPtrs pp{};
  for (int i = 0; i < (multicast ? 1 : world); ++i) pp.p[i] = const_cast<void*>(grads[i]);
  long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (multicast)
    sb::dp_reduce_shard_kernel<true><<<(int)blocks, 256, 0, s>>>(pp, world, rank, (size_t)off, (size_t)n, out, partials, status);
  else
    sb::dp_reduce_shard_kernel<false><<<(int)blocks, 256, 0, s>>>(pp, world, rank, (size_t)off, (size_t)n, out, partials, status);
  sb::dp_sum_partials_kernel<<<1, 256, 0, s>>>(partials, (int)blocks, ctl, 0, status);
  return (int)cudaGetLastError();
}

// params: `world` pointers to every rank's bf16 parameter buffer, or one multicast address with multicast != 0.
extern "C" int sb_dp_adam_bcast(float* master, float* m, float* v, const float* g, const void* const* params, int world,
                                int rank, int multicast, long off, long n, float lr, float beta1, float beta2, float eps,
                                float wd, float bc1, float bc2, float grad_scale, float max_norm, const float* ctl,
                                int stateless, cudaStream_t s) {
  if (n == 0) return 0;
  if (world < 1 || world > 8 || (n & 7) || (off & 7)) return (int)cudaErrorInvalidValue;
  sb::PeerPtrs pp{};
  for (int i = 0; i < (multicast ? 1 : world); ++i) pp.p[i] = const_cast<void*>(params[i]);
  sb::DpAdamArgs a{lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, max_norm};
  long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (multicast)
    sb::dp_adam_bcast_kernel<true><<<(int)blocks, 256, 0, s>>>(master, m, v, g, pp, world, rank, (size_t)off, (size_t)n, a,
                                                              ctl, stateless);
  else
    sb::dp_adam_bcast_kernel<false><<<(int)blocks, 256, 0, s>>>(master, m, v, g, pp, world, rank, (size_t)off, (size_t)n, a,
                                                               ctl, stateless);
  return (int)cudaGetLastError();
}
