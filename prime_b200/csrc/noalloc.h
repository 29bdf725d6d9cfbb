// Allocation-free entry point of the kernel library. It has no counterpart in the reference
// project: it exists for callers of this library that are not allowed to allocate device memory.
//
// Who those callers are: code that runs where cudaMalloc is off limits — inside a region whose
// memory budget was fixed up front (a serving process that pre-reserved all of HBM, a plugin
// loaded into somebody else's process), on a path that must not synchronise or touch the
// allocator for latency reasons, or from a host language binding that only passes raw pointers
// and has no allocator to hand a scratch buffer from. The regular entry point,
// pb_rmsnorm_bwd, makes such a caller provide a [ctas x N] fp32 scratch matrix for the partial
// weight-gradient sums; this variant keeps that scratch inside the library instead.
//
// How: the scratch is a file-scope `static __device__` array in elementwise_noalloc.cu, sized for
// the largest supported row width (PB_NOALLOC_MAX_N). Every GPU that loads the library carries
// that array (pb_rmsnorm_bwd_ctas() * PB_NOALLOC_MAX_N * 4 bytes, about 1.2 MB) until the process
// exits. The caller still passes every input and output buffer.
//
// Rules for the caller:
//   * N must be a multiple of 256 and at most PB_NOALLOC_MAX_N; wider rows are refused with
//     PB_NOALLOC_ERR_TOO_WIDE and nothing is launched. Other bad arguments give
//     PB_NOALLOC_ERR_BAD_ARG. pb_noalloc_strerror() turns a code into text.
//   * The first call on a device looks up the device address of the scratch array (one
//     cudaGetSymbolAddress, no allocation). Make that first call outside of any stream capture.
//   * All calls on a device share the one scratch array. The kernel overwrites every partial it
//     later reads, so nothing needs clearing between calls, but two calls that overlap on the GPU
//     (different streams, no ordering between them) race on it. Order them.
//   * No cudaMalloc, cudaFree or other allocating routine runs on this path.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define PB_NOALLOC_MAX_N 1024
#define PB_NOALLOC_ERR_BAD_ARG (-1)
#define PB_NOALLOC_ERR_TOO_WIDE (-3)
#define PB_NOALLOC_ERR_SETUP (-4)
#define PB_NOALLOC_ERR_LAUNCH (-30)

// dx = d(rmsnorm)/dx (+ dres if not null);  dw (+)= sum over rows of dy * x * rstd.
// x, w, dy, dres, dx: bf16; rstd: fp32 [M]; dw: bf16 or fp32 [N]. Returns 0 on success.
int pb_rmsnorm_bwd_noalloc(const void* x, const void* w, const float* rstd, const void* dy, const void* dres, void* dx,
                           void* dw, int dw_fp32, int dw_accumulate, int M, int N, void* stream);

const char* pb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
