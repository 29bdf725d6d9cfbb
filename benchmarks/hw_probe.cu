// Hardware probes behind the kernel designs of this package (sm_100a): each is a tiny kernel that times
// one thing with clock64 on an otherwise idle SM and returns cycles. Every wait is bounded.
//   umma_bench : issue / completion rate of the tcgen05.mma shapes used by the GEMM and attention kernels
//   prim_bench : latency of the synchronisation primitives (mbarrier ops, tcgen05.ld, fences, bulk waits)
//   wake_bench : latency from an mbarrier arrive to the waiter resuming, for three ways of waiting
//   xu_bench   : issue interval of special-function and conversion instructions per SM sub-partition
// Run through benchmarks/hw_probe.py.
#include "../prime_b200/csrc/common.cuh"
using namespace pb;
__global__ void __launch_bounds__(64, 1) umma_bench(int mode, int reps, unsigned long long* out, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    __shared__ uint64_t bar;
    __shared__ uint32_t tslot;
    __shared__ int abortf;
    for (int i = threadIdx.x; i < 160 * 1024 / 16; i += blockDim.x) reinterpret_cast<uint4*>(gen)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); abortf = 0; mbar_fence_init(); }
    if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tslot), 512); tmem_relinquish(); }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = tslot;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        constexpr uint32_t id_s = umma_idesc_bf16(128, 128, 0, 0);
        constexpr uint32_t id_kv = umma_idesc_bf16(128, 64, 1, 1);
        constexpr uint32_t id_dq = umma_idesc_bf16(128, 64, 0, 1);
        constexpr uint32_t id_g = umma_idesc_bf16(128, 256, 0, 0);
        constexpr uint32_t id_kk = umma_idesc_bf16(128, 64, 0, 0);
        const uint32_t A = base, B = base + 65536;
        long long t0 = clock64(), t1 = t0;
        int n_mma = 0;
        if (lane == 0) {
            for (int r = 0; r < reps; ++r) {
                if (mode == 0) {
                    for (int k = 0; k < 4; ++k) { const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
                        umma_f16_ss(tm, umma_smem_desc(A + off, 16, 1024), umma_smem_desc(B + off, 16, 1024), id_s, 1u); }
                    n_mma += 4;
                } else if (mode == 1) {
                    for (int k = 0; k < 8; ++k)
                        umma_f16_ss(tm + 256, umma_smem_desc(A + k * 2048, 16384, 1024), umma_smem_desc(B + k * 2048, 16384, 1024), id_kv, 1u);
                    n_mma += 8;
                } else if (mode == 2) {
                    for (int k = 0; k < 8; ++k)
                        umma_f16_ss(tm + 384, umma_smem_desc(A + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024), umma_smem_desc(B + k * 2048, 16384, 1024), id_dq, 1u);
                    n_mma += 8;
                } else if (mode == 3) {
                    for (int k = 0; k < 4; ++k) { const uint32_t off = (k & 3) * 32;
                        umma_f16_ss(tm, umma_smem_desc(A + off, 16, 1024), umma_smem_desc(B + off, 16, 1024), id_g, 1u); }
                    n_mma += 4;
                } else if (mode == 5) {
                    for (int k = 0; k < 4; ++k) { const uint32_t off = (k & 3) * 32;
                        umma_f16_ss(tm + 256, umma_smem_desc(A + off, 16, 1024), umma_smem_desc(B + off, 16, 1024), id_kk, 1u); }
                    n_mma += 4;
                } else {   // the per-pair mix of the backward kernel
                    for (int k = 0; k < 4; ++k) { const uint32_t off = (k & 3) * 32;
                        umma_f16_ss(tm, umma_smem_desc(A + off, 16, 1024), umma_smem_desc(B + off, 16, 1024), id_s, 1u); }
                    for (int k = 0; k < 4; ++k) { const uint32_t off = (k & 3) * 32;
                        umma_f16_ss(tm + 128, umma_smem_desc(A + 16384 + off, 16, 1024), umma_smem_desc(B + 16384 + off, 16, 1024), id_s, 1u); }
                    for (int k = 0; k < 8; ++k)
                        umma_f16_ss(tm + 256, umma_smem_desc(A + 32768 + k * 2048, 16384, 1024), umma_smem_desc(B + k * 2048, 16384, 1024), id_kv, 1u);
                    for (int k = 0; k < 8; ++k)
                        umma_f16_ss(tm + 320, umma_smem_desc(A + 32768 + k * 2048, 16384, 1024), umma_smem_desc(B + 32768 + k * 2048, 16384, 1024), id_kv, 1u);
                    for (int k = 0; k < 8; ++k)
                        umma_f16_ss(tm + 384, umma_smem_desc(A + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024), umma_smem_desc(B + k * 2048, 16384, 1024), id_dq, 1u);
                    n_mma += 32;
                }
            }
            umma_commit(smem_u32(&bar));
            t1 = clock64();
        }
        __syncwarp();
        bool ok = mbar_wait(smem_u32(&bar), 0, &abortf, status, PB_ERR_TIMEOUT_MISC);
        ok = __all_sync(0xffffffffu, ok);
        const long long t2 = clock64();
        if (lane == 0 && blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; out[2] = n_mma; }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}
extern "C" int umma_bench_run(int mode, int reps, int grid, unsigned long long* out_host, int* status) {
    static unsigned long long* d = nullptr;
    if (!d) cudaMalloc(&d, 64);
    cudaFuncSetAttribute(umma_bench, cudaFuncAttributeMaxDynamicSharedMemorySize, 161 * 1024);
    umma_bench<<<grid, 64, 161 * 1024>>>(mode, reps, d, status);
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    cudaMemcpy(out_host, d, 24, cudaMemcpyDeviceToHost);
    return 0;
}
#define T0 long long t_ = clock64()
#define T1(i) do { long long u_ = clock64(); if (lane == 0) acc[i] += u_ - t_; t_ = u_; } while (0)
__global__ void __launch_bounds__(128, 1) prim_bench(int spin, int reps, long long* out, float* gsrc, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    __shared__ uint64_t bar_done, bar_never, bar_cnt;
    __shared__ uint32_t tslot;
    __shared__ volatile int stop;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar_done), 1); mbar_init(smem_u32(&bar_never), 1); mbar_init(smem_u32(&bar_cnt), 1);
        stop = 0; mbar_fence_init();
        mbar_arrive(smem_u32(&bar_done));   // phase 0 of bar_done is complete
    }
    if (warp == 0) { tmem_alloc(smem_u32(&tslot), 128); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = tslot;
    long long acc[12];
    for (int i = 0; i < 12; ++i) acc[i] = 0;
    if (warp == 0) {
        uint32_t v[32];
        float sink = 0.f;
        for (int r = 0; r < reps; ++r) {
            T0;
            T1(0);                                                          // clock pair
            bool ok = mbar_try_wait(smem_u32(&bar_done), 0); T1(1);          // try_wait on a complete phase
            ok = __all_sync(0xffffffffu, ok); T1(2);                         // vote
            if (lane == 0) mbar_arrive(smem_u32(&bar_cnt)); __syncwarp(); T1(3);   // arrive
            tmem_ld32(tm + (uint32_t(0) << 16), v); tmem_ld_wait(); T1(4);   // tcgen05.ld x32 + wait
            sink += __uint_as_float(v[lane & 31 ? 3 : 5]);
#pragma unroll
            for (int q = 0; q < 16; ++q)
                *reinterpret_cast<uint4*>(gen + (q >> 3) * 16384 + lane * 128 + (((q & 7) ^ (lane & 7)) << 4)) = make_uint4(v[q], v[q + 1], r, q);
            T1(5);                                                          // 16 st.shared.v4
            fence_proxy_async_smem(); T1(6);                                 // fence.proxy.async after stores
            tc_fence_before(); T1(7);
            if (lane == 0) tma_store_wait_read<0>(); __syncwarp(); T1(8);    // bulk wait_group.read, nothing pending
            float g = gsrc[(r * 977 + lane * 64) & 0xfffff]; sink += g; T1(9);   // dependent global load (L2)
            if (!ok) sink += 1.f;
        }
        if (sink == 12345.f) out[100] = 1;
        stop = 1;
        if (lane == 0 && blockIdx.x == 0) for (int i = 0; i < 12; ++i) out[i] = acc[i];
    } else if (warp <= spin) {
        // spinning waiter, like a producer warp waiting for a free stage
        while (!stop) { if (mbar_try_wait(smem_u32(&bar_never), 0)) break; }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) { tc_fence_after(); tmem_dealloc(tm, 128); }
}
extern "C" int prim_bench_run(int spin, int reps, long long* out_host, float* gsrc, int* status) {
    static long long* d = nullptr;
    if (!d) cudaMalloc(&d, 1024);
    cudaMemset(d, 0, 1024);
    cudaFuncSetAttribute(prim_bench, cudaFuncAttributeMaxDynamicSharedMemorySize, 40 * 1024);
    prim_bench<<<1, 128, 40 * 1024>>>(spin, reps, d, gsrc, status);
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    cudaMemcpy(out_host, d, 96, cudaMemcpyDeviceToHost);
    return 0;
}
__device__ __forceinline__ bool test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred P;\n\tmbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\tselp.u32 %0, 1, 0, P;\n\t}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred P;\n\tmbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, P;\n\t}\n" : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
__global__ void __launch_bounds__(64, 1) wake_bench(int mode, int reps, int delay, long long* out) {
    __shared__ uint64_t bar_a, bar_b;
    __shared__ volatile long long t_arrive;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar_a), 1); mbar_init(smem_u32(&bar_b), 1); mbar_fence_init(); }
    __syncthreads();
    long long acc = 0, worst = 0;
    for (int r = 0; r < reps; ++r) {
        const uint32_t ph = r & 1;
        if (warp == 0) {
            // waiter on bar_a
            bool done = false;
            for (int i = 0; i < 4000000 && !done; ++i)
                done = mode == 0 ? mbar_try_wait(smem_u32(&bar_a), ph) : mode == 1 ? test_wait(smem_u32(&bar_a), ph) : try_wait_hint(smem_u32(&bar_a), ph, 32);
            const long long t = clock64();
            const long long d = t - t_arrive;
            acc += d; worst = d > worst ? d : worst;
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_b));   // hand back
        } else {
            // arriver: waits a while so that the waiter is parked, then arrives
            const long long t0 = clock64();
            while (clock64() - t0 < delay) {}
            if (lane == 0) { t_arrive = clock64(); mbar_arrive(smem_u32(&bar_a)); }
            __syncwarp();
            bool done = false;
            for (int i = 0; i < 4000000 && !done; ++i) done = test_wait(smem_u32(&bar_b), ph);
        }
    }
    if (threadIdx.x == 0) { out[0] = acc; out[1] = worst; }
}
extern "C" int wake_bench_run(int mode, int reps, int delay, long long* out_host) {
    static long long* d = nullptr;
    if (!d) cudaMalloc(&d, 64);
    wake_bench<<<1, 64>>>(mode, reps, delay, d);
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    cudaMemcpy(out_host, d, 16, cudaMemcpyDeviceToHost);
    return 0;
}
template <int OP>
__global__ void __launch_bounds__(256, 1) xu_bench(int reps, long long* out, float seed) {
    float x[16];
    uint32_t u[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) { x[i] = seed * (i + 1) + threadIdx.x * 1e-3f; u[i] = __float_as_uint(x[i]); }
    __syncthreads();
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (OP == 0) asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(x[i]));
            if (OP == 1) asm volatile("ex2.approx.ftz.bf16x2 %0, %0;" : "+r"(u[i]));
            if (OP == 2) { asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(u[i]) : "f"(x[i]), "f"(x[i])); x[i] = __uint_as_float(u[i]); }
            if (OP == 3) asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+f"(x[i]) : "f"(seed));
            if (OP == 4) asm volatile("ex2.approx.f16x2 %0, %0;" : "+r"(u[i]));
            if (OP == 5) asm volatile("max.f32 %0, %0, %1;" : "+f"(x[i]) : "f"(seed));
            if (OP == 6) asm volatile("fma.rn.bf16x2 %0, %0, %1, %1;" : "+r"(u[i]) : "r"(u[(i + 1) & 15]));
        }
    }
    const long long t1 = clock64();
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc += x[i] + __uint_as_float(u[i]);
    if (acc == 123.456f) out[8] = 1;
    if (threadIdx.x == 0 && blockIdx.x == 0) out[OP] = t1 - t0;
}
extern "C" int xu_bench_run(int reps, long long* host) {
    long long* d; cudaMalloc(&d, 128); cudaMemset(d, 0, 128);
    xu_bench<0><<<1, 256>>>(reps, d, 0.37f); xu_bench<1><<<1, 256>>>(reps, d, 0.37f); xu_bench<2><<<1, 256>>>(reps, d, 0.37f);
    xu_bench<3><<<1, 256>>>(reps, d, 0.37f); xu_bench<4><<<1, 256>>>(reps, d, 0.37f); xu_bench<5><<<1, 256>>>(reps, d, 0.37f);
    xu_bench<6><<<1, 256>>>(reps, d, 0.37f);
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    cudaMemcpy(host, d, 64, cudaMemcpyDeviceToHost); cudaFree(d);
    return 0;
}
