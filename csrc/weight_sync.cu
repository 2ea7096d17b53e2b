// Device-side weight movement for the trainer -> rollout-engine sync.
//
//   sb_multi_copy     any number of (src, dst, bytes) copies in one launch. The bytes of all pairs form one virtual
//                     range that is cut into 64 KiB pieces; CTA b handles pieces b, b + grid, ... and finds the pair a
//                     piece belongs to by binary search over the prefix sums it builds in shared memory. 16-byte
//                     vector path when both pointers of a pair are 16-byte aligned, byte path for the ragged rest.
//                     dst may be peer-mapped memory of another GPU (plain stores over NVLink).
#include "common.cuh"

namespace sb {

constexpr int MC_THREADS = 256;
constexpr long long MC_PIECE = 64 * 1024;
constexpr int MC_MAX_PAIRS = 4096;

__global__ void __launch_bounds__(MC_THREADS)
multi_copy_kernel(const long long* __restrict__ src, const long long* __restrict__ dst, const long long* __restrict__ bytes,
                  int n) {
  extern __shared__ long long prefix[];  // n + 1 piece offsets
  if (threadIdx.x == 0) {
    long long acc = 0;
    for (int i = 0; i < n; ++i) {
      prefix[i] = acc;
      acc += (bytes[i] + MC_PIECE - 1) / MC_PIECE;
    }
    prefix[n] = acc;
  }
  __syncthreads();
  const long long pieces = prefix[n];
  for (long long pc = blockIdx.x; pc < pieces; pc += gridDim.x) {
    int lo = 0, hi = n - 1;  // last pair whose first piece is <= pc
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (prefix[mid] <= pc) lo = mid; else hi = mid - 1;
    }
    const long long off = (pc - prefix[lo]) * MC_PIECE;
    const long long len = min(MC_PIECE, bytes[lo] - off);
    const char* s = reinterpret_cast<const char*>(src[lo]) + off;
    char* d = reinterpret_cast<char*>(dst[lo]) + off;
    if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 15) == 0) {
      const long long nv = len >> 4;
      const uint4* sv = reinterpret_cast<const uint4*>(s);
      uint4* dv = reinterpret_cast<uint4*>(d);
      for (long long i = threadIdx.x; i < nv; i += MC_THREADS) dv[i] = sv[i];
      for (long long i = (nv << 4) + threadIdx.x; i < len; i += MC_THREADS) d[i] = s[i];
    } else {
      for (long long i = threadIdx.x; i < len; i += MC_THREADS) d[i] = s[i];
    }
  }
}

}  // namespace sb

// src / dst / bytes: device arrays of n 64-bit entries (addresses as integers). total_bytes only sizes the grid.
extern "C" int sb_multi_copy(const void* src, const void* dst, const void* bytes, int n, long total_bytes, int num_sms,
                             cudaStream_t s) {
  if (n <= 0) return 0;
  if (n > sb::MC_MAX_PAIRS) {
    sb::set_last_error("sb_multi_copy: more than 4096 pairs in one call");
    return (int)cudaErrorInvalidValue;
  }
  long long pieces = total_bytes / sb::MC_PIECE + n;
  const int grid = (int)(pieces < (long long)num_sms * 8 ? pieces : (long long)num_sms * 8);
  sb::multi_copy_kernel<<<grid > 0 ? grid : 1, sb::MC_THREADS, (n + 1) * sizeof(long long), s>>>(
      (const long long*)src, (const long long*)dst, (const long long*)bytes, n);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------------------
//   sb_multi_copy_2d  any number of strided 2-D copies in one launch: pair i moves rows[i] rows of row_bytes[i] bytes
//                     from src[i] (pitch src_pitch[i]) to dst[i] (pitch dst_pitch[i]). This is the gather + re-layout
//                     step of a weight sync between different tensor-parallel shardings: a destination tensor in the
//                     engine's layout is the union of row ranges (column-parallel weights, with the fused QKV / gate-up
//                     orders handled by giving each of q, k, v, gate, up its own pair) or column ranges (row-parallel
//                     weights: row_bytes < dst_pitch) of the source ranks' shards, which may live on other GPUs and
//                     are then read with plain loads over NVLink. Work is cut into (pair, block of rows) pieces of about
//                     64 KiB striped over the CTAs. Pointers and row_bytes must be multiples of 16 bytes.
namespace sb {

struct Copy2D {
  long long src, dst, rows, row_bytes, src_pitch, dst_pitch;
};

__global__ void __launch_bounds__(MC_THREADS)
multi_copy_2d_kernel(const Copy2D* __restrict__ tab, int n) {
  extern __shared__ long long prefix[];  // n + 1 piece offsets
  __shared__ long long rows_per_piece_s;
  if (threadIdx.x == 0) {
    long long acc = 0;
    for (int i = 0; i < n; ++i) {
      prefix[i] = acc;
      const long long rpp = max(1LL, MC_PIECE / max(16LL, tab[i].row_bytes));
      acc += (tab[i].rows + rpp - 1) / rpp;
    }
    prefix[n] = acc;
  }
  __syncthreads();
  const long long pieces = prefix[n];
  for (long long pc = blockIdx.x; pc < pieces; pc += gridDim.x) {
    int lo = 0, hi = n - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (prefix[mid] <= pc) lo = mid; else hi = mid - 1;
    }
    const Copy2D c = tab[lo];
    const long long rpp = max(1LL, MC_PIECE / max(16LL, c.row_bytes));
    const long long r0 = (pc - prefix[lo]) * rpp, r1 = min(c.rows, r0 + rpp);
    const long long vec_per_row = c.row_bytes >> 4;
    const long long total = (r1 - r0) * vec_per_row;
    for (long long i = threadIdx.x; i < total; i += MC_THREADS) {
      const long long r = r0 + i / vec_per_row, v = i % vec_per_row;
      const uint4 val = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(c.src) + r * c.src_pitch + (v << 4));
      *reinterpret_cast<uint4*>(reinterpret_cast<char*>(c.dst) + r * c.dst_pitch + (v << 4)) = val;
    }
  }
}

}  // namespace sb

// table: device array of n entries of six 64-bit integers {src, dst, rows, row_bytes, src_pitch, dst_pitch}.
extern "C" int sb_multi_copy_2d(const void* table, int n, long total_bytes, int num_sms, cudaStream_t s) {
  if (n <= 0) return 0;
  if (n > sb::MC_MAX_PAIRS) {
    sb::set_last_error("sb_multi_copy_2d: more than 4096 pairs in one call");
    return (int)cudaErrorInvalidValue;
  }
  long long pieces = total_bytes / sb::MC_PIECE + n;
  const int grid = (int)(pieces < (long long)num_sms * 8 ? pieces : (long long)num_sms * 8);
  sb::multi_copy_2d_kernel<<<grid > 0 ? grid : 1, sb::MC_THREADS, (n + 1) * sizeof(long long), s>>>(
      static_cast<const sb::Copy2D*>(table), n);
  return (int)cudaGetLastError();
}
