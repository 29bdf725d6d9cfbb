// Allocation-free variant of the RMSNorm backward entry point; see noalloc.h for who needs it and
// the rules that come with it. Same kernels as pb_rmsnorm_bwd; only the home of the fp32 partial
// sums differs: a static device array owned by this file instead of a caller-provided buffer.
#include "noalloc.h"
#include "rmsnorm_bwd.cuh"
#include <mutex>

extern "C" int pb_rmsnorm_bwd_ctas();

namespace {

constexpr int kMaxCtas = 148 * 2;
constexpr int kMaxDevices = 64;

// [ctas][N] fp32 partial weight-gradient sums. In host code this name is only a handle for the
// runtime, never a device address: the address is fetched once per device below.
static __device__ __align__(256) float g_rms_bwd_partials[kMaxCtas * PB_NOALLOC_MAX_N];

float* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mutex;

// Device address of the scratch array on the current device (looked up on first use).
int scratch_for_current_device(float** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return PB_NOALLOC_ERR_SETUP;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        float* p = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rms_bwd_partials) != cudaSuccess || p == nullptr) {
            cudaGetLastError();
            return PB_NOALLOC_ERR_SETUP;
        }
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return 0;
}

}  // namespace

extern "C" const char* pb_noalloc_strerror(int code) {
    switch (code) {
        case 0: return "ok";
        case PB_NOALLOC_ERR_BAD_ARG: return "bad argument: N must be a positive multiple of 256, M positive, pointers non-null";
        case PB_NOALLOC_ERR_TOO_WIDE: return "row width N exceeds PB_NOALLOC_MAX_N, the size the built-in scratch array was compiled for";
        case PB_NOALLOC_ERR_SETUP: return "could not obtain the device address of the built-in scratch array on this device";
        case PB_NOALLOC_ERR_LAUNCH: return "kernel launch failed";
        default: return "unknown error";
    }
}

extern "C" int pb_rmsnorm_bwd_noalloc(const void* x, const void* w, const float* rstd, const void* dy, const void* dres, void* dx,
                                      void* dw, int dw_fp32, int dw_accumulate, int M, int N, void* stream) {
    using namespace pb;
    if (!x || !w || !rstd || !dy || !dx || !dw || M <= 0 || N <= 0 || (N % 256) != 0) return PB_NOALLOC_ERR_BAD_ARG;
    if (N > PB_NOALLOC_MAX_N) return PB_NOALLOC_ERR_TOO_WIDE;
    const int ctas = pb_rmsnorm_bwd_ctas();
    if (ctas > kMaxCtas) return PB_NOALLOC_ERR_SETUP;
    float* partials = nullptr;
    if (int rc = scratch_for_current_device(&partials)) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w; auto DY = (const __nv_bfloat16*)dy;
    auto DR = (const __nv_bfloat16*)dres; auto DX = (__nv_bfloat16*)dx;
    switch (N / 256) {
        case 1: rmsnorm_bwd_kernel<1><<<ctas, 256, 0, st>>>(X, W, rstd, DY, DR, DX, partials, M); break;
        case 2: rmsnorm_bwd_kernel<2><<<ctas, 256, 0, st>>>(X, W, rstd, DY, DR, DX, partials, M); break;
        case 3: rmsnorm_bwd_kernel<3><<<ctas, 256, 0, st>>>(X, W, rstd, DY, DR, DX, partials, M); break;
        case 4: rmsnorm_bwd_kernel<4><<<ctas, 256, 0, st>>>(X, W, rstd, DY, DR, DX, partials, M); break;
        default: return PB_NOALLOC_ERR_BAD_ARG;
    }
    if (cudaGetLastError() != cudaSuccess) return PB_NOALLOC_ERR_LAUNCH;
    // every one of the ctas*N partials was just rewritten by the kernel above, so stale contents of
    // the shared array from an earlier call never reach this reduction
    colsum_partials_kernel<<<(N + 31) / 32, 256, 0, st>>>(partials, dw, ctas, N, dw_fp32, dw_accumulate);
    return cudaGetLastError() == cudaSuccess ? 0 : PB_NOALLOC_ERR_LAUNCH;
}
