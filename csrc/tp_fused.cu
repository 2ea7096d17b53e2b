// Tensor-parallel all-reduce fused with the residual add and the RMSNorm that always follow it in a decoder layer
// (after the attention output projection and after the MLP down projection), over NVLink peer memory:
//
//   partial_r [T, H] bf16   this rank's row-parallel GEMM output, in a symmetric buffer every rank can read
//   h   = sum_r partial_r + residual          (fp32; written back as the new residual, bf16)
//   y   = h * rsqrt(mean(h^2) + eps) * w      (bf16)
//
// One-shot scheme, sized for decode batches: every rank computes all T rows itself, reading the peers' partial rows
// either with plain P2P loads (summed in rank order, so every rank gets bit-identical results) or with one
// multimem.ld_reduce per 16 bytes through the NVSwitch multicast address (the switch does the sum). Nothing is written
// to a peer. Each CTA runs its own bounded flag barrier with the same CTA of every peer before it reads (the flag of a
// peer's CTA is only raised after that peer's producing GEMM has finished, by stream order), so there is no separate
// barrier launch and no NCCL call. The epoch of CTA b lives in device memory and is advanced by the CTA itself: the
// launch arguments never change, so the kernel can be captured in a CUDA graph and replayed.
//
// The caller alternates between two partial buffers and places one full barrier (sb_symm_barrier) at the start of each
// forward pass; that is what makes it safe for a fast rank to start the next GEMM while a slow one is still reading.
// Every wait is bounded (sb_set_peer_wait_limit_ns, 2 s unless changed): on expiry the CTA records a status word, skips
// its rows and returns; later launches see the status word and return at once (see the kernel).
#include "common.cuh"

namespace sb {

struct TpPeerPtrs {
  void* p[8];
};

__device__ __forceinline__ void tp_st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t tp_ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
// 8 bf16 summed over all ranks by the switch, accumulated in fp32
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}

constexpr int TP_THREADS = 256;
constexpr int TP_MAX_VEC = 4;      // 8-element vectors per thread -> H <= 8192
constexpr int TP_MAX_BLOCKS = 148;

// flags: every rank's flag array, [TP_MAX_BLOCKS][8] words; word [b][r] on rank q = last epoch rank r's CTA b announced
// to q. epochs: this rank's own [TP_MAX_BLOCKS] counters.
template <bool MC>
__global__ void __launch_bounds__(TP_THREADS)
tp_ar_add_rmsnorm_kernel(TpPeerPtrs partial, TpPeerPtrs flags, uint32_t* __restrict__ epochs,
                         const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ w,
                         __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ res_out, int T, int H, float eps,
                         int rank, int world, int* status, unsigned long long limit_ns) {
  __shared__ float scratch[32];
  __shared__ int s_ok;
  const int b = blockIdx.x, tid = threadIdx.x;
  // A non-zero status word (an earlier wait of this process gave up) is sticky: the flag is still raised so that the
  // peers are not held up, but this CTA neither waits nor produces rows; the host sees the status and raises.
  if (tid == 0) s_ok = (status == nullptr || *reinterpret_cast<volatile int*>(status) == 0) ? 1 : 0;
  __syncthreads();
  const bool failed = s_ok == 0;
  if (tid < world) {
    const uint32_t epoch = epochs[b] + 1;  // every thread < world reads the old value before thread 0 stores the new one
    __syncwarp((1u << world) - 1u);
    if (tid == 0) epochs[b] = epoch;
    __threadfence_system();
    tp_st_release_sys(static_cast<uint32_t*>(flags.p[tid]) + b * 8 + rank, epoch);
    const uint32_t* mine = static_cast<const uint32_t*>(flags.p[rank]) + b * 8 + tid;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t it = 0;
    while (!failed && static_cast<int32_t>(tp_ld_acquire_sys(mine) - epoch) < 0) {
      if ((++it & 0xff) == 0 && globaltimer_ns() - t0 > limit_ns) {
        if (status) atomicCAS(status, 0, ERR_WAIT_PEER | (tid << 8));
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;

  const int nvec = H >> 3;
  const float inv_h = 1.f / static_cast<float>(H);
  for (int row = b; row < T; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * H;
    float v[TP_MAX_VEC][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < TP_MAX_VEC; ++j) {
      const int c = tid + j * TP_THREADS;
      if (c < nvec) {
        float acc[8];
        if constexpr (MC) {
          const uint4 u = multimem_ld_reduce_bf16x8(static_cast<const __nv_bfloat16*>(partial.p[0]) + base + c * 8);
          float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
          acc[0] = a0.x; acc[1] = a0.y; acc[2] = a1.x; acc[3] = a1.y; acc[4] = a2.x; acc[5] = a2.y; acc[6] = a3.x; acc[7] = a3.y;
        } else {
          uint4 u[8];
#pragma unroll
          for (int r = 0; r < 8; ++r)  // all peers' loads in flight together
            if (r < world) u[r] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(partial.p[r]) + base + c * 8);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
          for (int r = 0; r < 8; ++r)
            if (r < world) {
              float2 a0 = unpack_bf16x2(u[r].x), a1 = unpack_bf16x2(u[r].y), a2 = unpack_bf16x2(u[r].z), a3 = unpack_bf16x2(u[r].w);
              acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y;
              acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
            }
        }
        if (residual != nullptr) {
          const uint4 ru = *reinterpret_cast<const uint4*>(residual + base + c * 8);
          float2 a0 = unpack_bf16x2(ru.x), a1 = unpack_bf16x2(ru.y), a2 = unpack_bf16x2(ru.z), a3 = unpack_bf16x2(ru.w);
          acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y; acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          v[j][i] = acc[i];
          ss += acc[i] * acc[i];
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(res_out + base + c * 8) = o;
      }
    }
    const float rstd = rsqrtf(block_sum<TP_THREADS>(ss, scratch) * inv_h + eps);
#pragma unroll
    for (int j = 0; j < TP_MAX_VEC; ++j) {
      const int c = tid + j * TP_THREADS;
      if (c < nvec) {
        const uint4 gu = *reinterpret_cast<const uint4*>(w + c * 8);
        float2 g0 = unpack_bf16x2(gu.x), g1 = unpack_bf16x2(gu.y), g2 = unpack_bf16x2(gu.z), g3 = unpack_bf16x2(gu.w);
        uint4 o;
        o.x = pack_bf16x2(v[j][0] * rstd * g0.x, v[j][1] * rstd * g0.y);
        o.y = pack_bf16x2(v[j][2] * rstd * g1.x, v[j][3] * rstd * g1.y);
        o.z = pack_bf16x2(v[j][4] * rstd * g2.x, v[j][5] * rstd * g2.y);
        o.w = pack_bf16x2(v[j][6] * rstd * g3.x, v[j][7] * rstd * g3.y);
        *reinterpret_cast<uint4*>(y + base + c * 8) = o;
      }
    }
  }
}

}  // namespace sb

// partial: `world` pointers to every rank's partial buffer (own included), or, with multicast != 0, the multicast
// address in partial[0]. flags: `world` pointers to every rank's flag array (148 x 8 words, zeroed once). epochs: this
// rank's 148 counters (zeroed once). residual may be null (first use in a forward pass). Returns a CUDA error code.
extern "C" int sb_tp_ar_add_rmsnorm(const void* const* partial, const void* const* flags, unsigned* epochs,
                                    const void* residual, const void* w, void* y, void* res_out, int T, int H, float eps,
                                    int rank, int world, int multicast, int* status, cudaStream_t s) {
  using bf16 = __nv_bfloat16;
  if (T == 0) return 0;
  if (world < 2 || world > 8 || rank < 0 || rank >= world || (H & 7) || H > sb::TP_THREADS * sb::TP_MAX_VEC * 8)
    return (int)cudaErrorInvalidValue;
  sb::TpPeerPtrs pp{}, ff{};
  for (int i = 0; i < (multicast ? 1 : world); ++i) pp.p[i] = const_cast<void*>(partial[i]);
  for (int i = 0; i < world; ++i) ff.p[i] = const_cast<void*>(flags[i]);
  // the grid depends only on T, which is the same on every rank of the group, so CTA b exists on all of them
  const int blocks = T < sb::TP_MAX_BLOCKS ? T : sb::TP_MAX_BLOCKS;
  if (multicast)
    sb::tp_ar_add_rmsnorm_kernel<true><<<blocks, sb::TP_THREADS, 0, s>>>(pp, ff, epochs, (const bf16*)residual, (const bf16*)w,
                                                                         (bf16*)y, (bf16*)res_out, T, H, eps, rank, world, status,
                                                                         sb::peer_wait_limit_ns());
  else
    sb::tp_ar_add_rmsnorm_kernel<false><<<blocks, sb::TP_THREADS, 0, s>>>(pp, ff, epochs, (const bf16*)residual, (const bf16*)w,
                                                                          (bf16*)y, (bf16*)res_out, T, H, eps, rank, world, status,
                                                                          sb::peer_wait_limit_ns());
  return (int)cudaGetLastError();
}
