// RMSNorm backward that never allocates: sb_rmsnorm_bwd_static.
//
// This entry point has no counterpart in the reference framework. It exists for callers that cannot allocate
// device memory at the moment they need the kernel: code running where the caching allocator must not be touched
// (inside a region being recorded for replay, inside an allocator callback, under a memory-saver pause that has
// handed the pool to another process) and plain C/C++ hosts that link this library without PyTorch and have no
// allocator to ask. The regular entry point, sb_rmsnorm_bwd, takes its `dw_partial` scratch from the caller, which
// in practice means one torch.empty per call; this one keeps the scratch inside the library instead.
//
// Same math as sb_rmsnorm_bwd (same kernels, same summation order for a given CTA count):
//     dh = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres_in),   dw (+)= sum_rows dy * xhat,   xhat = h * rstd
//
// Scratch. The per-CTA partial sums of dw live in one file-scope device array,
//     SB_RMSNORM_STATIC_MAX_CTAS x SB_RMSNORM_STATIC_MAX_H floats = 148 x 8192 x 4 B = 4.6 MiB per device,
// part of the library image. Every CTA overwrites its whole row before the reduction reads it, so nothing in the
// array has to be zero at entry and nothing is cleared between calls.
//
// Limits. H must be a multiple of 8 and at most SB_RMSNORM_STATIC_MAX_H; T is unbounded (rows are strided over at
// most SB_RMSNORM_STATIC_MAX_CTAS CTAs). dy, h, w, dres_in and dh must be 16-byte aligned (the kernels move eight
// bf16 values per access; with H a multiple of 8 every row then is too), rstd and dw 4-byte aligned. A call outside
// these limits launches nothing, returns cudaErrorInvalidValue (1) and leaves the reason in sb_last_error().
// sb_last_error() returns a buffer that belongs to the calling host thread: read it on the thread that made the
// failing call. The return value of a successful launch is whatever cudaGetLastError() reports after the second
// kernel has been queued, so an asynchronous error raised by unrelated earlier work on the device can surface here.
//
// Set-up. The array's device address is looked up once per device (cudaGetSymbolAddress) and cached. Call
// sb_rmsnorm_bwd_static_setup() with the device current to do that explicitly; otherwise the first
// sb_rmsnorm_bwd_static call on a device does it. The lookup is a synchronous runtime call that may load the
// library's device code, so make that first call (or the explicit set-up) before any stream capture begins.
//
// Sharing. All calls on a device use the same array. Calls issued to one stream are ordered and safe. Two calls
// that may overlap (different streams without an event between them, or two host threads on different streams)
// race on the scratch and produce a wrong dw; order them yourself.
//
// After set-up a call performs two kernel launches and nothing else: no cudaMalloc / cudaFree, no stream
// synchronisation, no library routine that allocates.
#ifndef SLIME_B200_RMSNORM_BWD_STATIC_H_
#define SLIME_B200_RMSNORM_BWD_STATIC_H_

#include <cuda_runtime_api.h>

#define SB_RMSNORM_STATIC_MAX_CTAS 148
#define SB_RMSNORM_STATIC_MAX_H 8192

#ifdef __cplusplus
extern "C" {
#endif

// Looks up and caches the scratch address for the current device. Returns 0 or a cudaError_t value.
int sb_rmsnorm_bwd_static_setup(void);

// dy, h, dres_in (may be null), dh: [T, H] bf16 row-major; w: [H] bf16; rstd: [T] fp32 (saved by the forward);
// dw: [H] fp32, overwritten, or added to when accumulate_dw != 0. Returns 0 or a cudaError_t value.
int sb_rmsnorm_bwd_static(const void* dy, const void* h, const void* w, const float* rstd, const void* dres_in,
                          void* dh, float* dw, int T, int H, int accumulate_dw, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif  // SLIME_B200_RMSNORM_BWD_STATIC_H_
