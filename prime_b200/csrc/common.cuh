// Shared device-side primitives for the sm_100a kernels of this package:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (alloc / mma / commit / ld) and
// bounded waits. Everything here is inline PTX; nothing depends on a library.
//
// Every spin in this package goes through a *bounded* wait: after a wall-clock
// budget (globaltimer) the waiter records an error code in a global status word,
// raises a CTA-wide abort flag in shared memory and returns false, so the kernel
// can tear down (free TMEM) and return instead of hanging the device.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace pb {

// ----------------------------------------------------------------------------
// error codes written to the status word (host reads them after the launch)
// ----------------------------------------------------------------------------
enum : int {
    PB_OK = 0,
    PB_ERR_TIMEOUT_FULL = 1,    // consumer never saw a TMA stage land
    PB_ERR_TIMEOUT_EMPTY = 2,   // producer never got a free stage
    PB_ERR_TIMEOUT_TMEM_FULL = 3,
    PB_ERR_TIMEOUT_TMEM_EMPTY = 4,
    PB_ERR_TIMEOUT_PEER = 5,    // a peer flag never reached the expected epoch
    PB_ERR_TIMEOUT_MISC = 6,
};

#ifndef PB_WAIT_BUDGET_NS
#define PB_WAIT_BUDGET_NS 2000000000ull  // 2 s per wait, then give up
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}\n"
        : "=r"(pred));
    return pred != 0;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait on an mbarrier phase. `abort_flag` lives in shared memory and is
// raised by whichever waiter runs out of budget first; every other waiter of the
// CTA notices it within a few hundred polls and gives up too.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
    // fast path: no timer reads (a %globaltimer read costs far more than a try_wait)
#pragma unroll 1
    for (int i = 0; i < 2048; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t polls = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++polls & 0x3ff) == 0) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > PB_WAIT_BUDGET_NS) {
                *abort_flag = 1;
                if (status) atomicCAS(status, 0, code | (int(blockIdx.x) << 8));
                return false;
            }
        }
    }
    return true;
}

// Work-item ring of a persistent CTA: one producer warp draws item numbers from a global counter and publishes
// them (-1 = no more work) into ring[k & 3]; every consumer warp (or single consumer thread) takes each entry once.
// bar_full[4] are initialised with count 1, bar_empty[4] with the number of consumers.
struct ItemRing {
    uint32_t bar_full, bar_empty;   // [4] each
    volatile int* ring;
    volatile int* abort_flag;
    int* status;
    // producer warp (all lanes call): draws the k-th item of this CTA and publishes it; returns it, or -2 on a timeout
    __device__ __forceinline__ int publish(int k, int* counter, int n_items) {
        const int slot = k & 3;
        bool ok = mbar_wait(bar_empty + 8 * slot, ((k >> 2) & 1) ^ 1, abort_flag, status, PB_ERR_TIMEOUT_EMPTY);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return -2;
        int idx = 0;
        if ((threadIdx.x & 31) == 0) {
            idx = atomicAdd(counter, 1);
            if (idx >= n_items) idx = -1;
            ring[slot] = idx;
            mbar_arrive(bar_full + 8 * slot);
        }
        return __shfl_sync(0xffffffffu, idx, 0);
    }
    // consumer warp (all lanes call): the k-th item of this CTA, or -2 on a timeout
    __device__ __forceinline__ int take(int k) {
        const int slot = k & 3;
        bool ok = mbar_wait(bar_full + 8 * slot, (k >> 2) & 1, abort_flag, status, PB_ERR_TIMEOUT_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return -2;
        const int idx = ring[slot];
        __syncwarp();
        if ((threadIdx.x & 31) == 0) mbar_arrive(bar_empty + 8 * slot);
        return idx;
    }
    // the same for a consumer that is a single thread
    __device__ __forceinline__ int take_thread(int k) {
        const int slot = k & 3;
        if (!mbar_wait(bar_full + 8 * slot, (k >> 2) & 1, abort_flag, status, PB_ERR_TIMEOUT_FULL)) return -2;
        const int idx = ring[slot];
        mbar_arrive(bar_empty + 8 * slot);
        return idx;
    }
};

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------------------------
// TMA (tiled bulk tensor copies). No cluster multicast anywhere in this package.
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src_smem, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src_smem), "r"(c0), "r"(c1)
        : "memory");
}
// element-wise add of a shared-memory tile into global memory (element type from the tensor map)
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, uint32_t src_smem, int c0, int c1) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src_smem), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------
// tcgen05: tensor memory + 5th-gen tensor core MMA (single-CTA group)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; bf16/f16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// A operand read from tensor memory (used by attention: P stays in TMEM).
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Four tcgen05.mma (cta_group::1, kind::f16, both operands in shared memory) in one instruction
// sequence. K-steps 1..3 use the descriptors of step 0 advanced by inc_a / inc_b in the 14-bit start
// address field (16-byte units). Up to two mbarriers are polled BEFORE the MMAs are issued and the
// poll results are consumed only AFTER them (and after the optional commits), so the latency of the
// polls is hidden behind the issue. A barrier address of 0 skips that commit / poll.
// Returns bit 0 / bit 1 = phase `par0` / `par1` of `peek0` / `peek1` has completed.
__device__ __forceinline__ uint32_t umma4_f16_ss_peek(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t inc_a,
                                                      uint32_t inc_b, uint32_t idesc, uint32_t acc_first,
                                                      uint32_t commit0, uint32_t commit1, uint32_t commit2,
                                                      uint32_t peek0, uint32_t par0, uint32_t peek1, uint32_t par1) {
    uint32_t r0, r1;
    asm volatile(
        "{\n\t"
        ".reg .pred P0, P1, K0, K1, Q, T, C0, C1, C2;\n\t"
        ".reg .b64 a1, a2, a3, b1, b2, b3, ia, ib;\n\t"
        "setp.ne.b32 K0, %13, 0;\n\t"
        "setp.ne.b32 K1, %15, 0;\n\t"
        "setp.ne.b32 P0, 0, 0;\n\t"
        "setp.ne.b32 P1, 0, 0;\n\t"
        "@K0 mbarrier.try_wait.parity.shared::cta.b64 P0, [%13], %14;\n\t"
        "@K1 mbarrier.try_wait.parity.shared::cta.b64 P1, [%15], %16;\n\t"
        "setp.ne.b32 Q, %8, 0;\n\t"
        "setp.eq.b32 T, 0, 0;\n\t"
        "setp.ne.b32 C0, %10, 0;\n\t"
        "setp.ne.b32 C1, %11, 0;\n\t"
        "setp.ne.b32 C2, %12, 0;\n\t"
        "cvt.u64.u32 ia, %5;\n\t"
        "cvt.u64.u32 ib, %6;\n\t"
        "add.s64 a1, %3, ia;\n\t"
        "add.s64 a2, a1, ia;\n\t"
        "add.s64 a3, a2, ia;\n\t"
        "add.s64 b1, %4, ib;\n\t"
        "add.s64 b2, b1, ib;\n\t"
        "add.s64 b3, b2, ib;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%2], %3, %4, %7, Q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%2], a1, b1, %7, T;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%2], a2, b2, %7, T;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%2], a3, b3, %7, T;\n\t"
        "@C0 tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%10];\n\t"
        "@C1 tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%11];\n\t"
        "@C2 tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%12];\n\t"
        "selp.u32 %0, 1, 0, P0;\n\t"
        "selp.u32 %1, 2, 0, P1;\n\t"
        "}\n"
        : "=r"(r0), "=r"(r1)
        : "r"(d_tmem), "l"(da), "l"(db), "r"(inc_a), "r"(inc_b), "r"(idesc), "r"(acc_first), "r"(0u), "r"(commit0),
          "r"(commit1), "r"(commit2), "r"(peek0), "r"(par0), "r"(peek1), "r"(par1)
        : "memory");
    return r0 | r1;
}
// Same as umma4_f16_ss_peek with the A operand in tensor memory (its address advances by inc_a
// columns per K-step).
__device__ __forceinline__ uint32_t umma4_f16_ts_peek(uint32_t d_tmem, uint32_t a_tmem, uint64_t db, uint32_t inc_a,
                                                      uint32_t inc_b, uint32_t idesc, uint32_t acc_first,
                                                      uint32_t commit0, uint32_t commit1, uint32_t commit2,
                                                      uint32_t peek0, uint32_t par0, uint32_t peek1, uint32_t par1) {
    uint32_t r0, r1;
    asm volatile(
        "{\n\t"
        ".reg .pred P0, P1, K0, K1, Q, T, C0, C1, C2;\n\t"
        ".reg .b64 b1, b2, b3, ib;\n\t"
        ".reg .b32 a1, a2, a3;\n\t"
        "setp.ne.b32 K0, %13, 0;\n\t"
        "setp.ne.b32 K1, %15, 0;\n\t"
        "setp.ne.b32 P0, 0, 0;\n\t"
        "setp.ne.b32 P1, 0, 0;\n\t"
        "@K0 mbarrier.try_wait.parity.shared::cta.b64 P0, [%13], %14;\n\t"
        "@K1 mbarrier.try_wait.parity.shared::cta.b64 P1, [%15], %16;\n\t"
        "setp.ne.b32 Q, %8, 0;\n\t"
        "setp.eq.b32 T, 0, 0;\n\t"
        "setp.ne.b32 C0, %10, 0;\n\t"
        "setp.ne.b32 C1, %11, 0;\n\t"
        "setp.ne.b32 C2, %12, 0;\n\t"
        "cvt.u64.u32 ib, %6;\n\t"
        "add.u32 a1, %3, %5;\n\t"
        "add.u32 a2, a1, %5;\n\t"
        "add.u32 a3, a2, %5;\n\t"
        "add.s64 b1, %4, ib;\n\t"
        "add.s64 b2, b1, ib;\n\t"
        "add.s64 b3, b2, ib;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%2], [%3], %4, %7, Q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%2], [a1], b1, %7, T;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%2], [a2], b2, %7, T;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%2], [a3], b3, %7, T;\n\t"
        "@C0 tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%10];\n\t"
        "@C1 tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%11];\n\t"
        "@C2 tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%12];\n\t"
        "selp.u32 %0, 1, 0, P0;\n\t"
        "selp.u32 %1, 2, 0, P1;\n\t"
        "}\n"
        : "=r"(r0), "=r"(r1)
        : "r"(d_tmem), "r"(a_tmem), "l"(db), "r"(inc_a), "r"(inc_b), "r"(idesc), "r"(acc_first), "r"(0u), "r"(commit0),
          "r"(commit1), "r"(commit2), "r"(peek0), "r"(par0), "r"(peek1), "r"(par1)
        : "memory");
    return r0 | r1;
}
// mbarrier arrives once all previously issued MMAs of this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// 32 lanes x 32 bit, N consecutive columns: thread i of the warp gets lane (base+i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
          "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
          "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------
// UMMA descriptors (bf16/f16, 128-byte swizzle, tiles whose base is 1024-B aligned)
// ----------------------------------------------------------------------------
// Shared-memory matrix descriptor: start address, leading/stride byte offsets
// (all >> 4), version 1 (Blackwell) at bit 46, swizzle mode 2 (=128 B) at bit 61.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= uint64_t((saddr >> 4) & 0x3fff);
    d |= uint64_t((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= uint64_t((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(2) << 61;
    return d;
}
// Instruction descriptor for kind::f16 with bf16 A/B and fp32 D.
// a_mn / b_mn: operand is MN-major (1) instead of K-major (0).
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N, int a_mn, int b_mn) {
    return (1u << 4)                      // D format: F32
           | (1u << 7)                    // A format: BF16
           | (1u << 10)                   // B format: BF16
           | (uint32_t(a_mn) << 15) | (uint32_t(b_mn) << 16)
           | (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

// ----------------------------------------------------------------------------
// packed fp32 pairs (Blackwell f32x2: one instruction, two fp32 lanes) and 3-input max
// ----------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long f32x2_pack(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f32x2_unpack(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long f32x2_fma(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ unsigned long long f32x2_add(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long f32x2_mul(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// ----------------------------------------------------------------------------
// misc numerics helpers
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
    return __bfloat1622float2(v);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace pb
