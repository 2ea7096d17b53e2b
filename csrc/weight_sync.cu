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
