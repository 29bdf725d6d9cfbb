// CTA-pair bf16 GEMM for sm_100a: tcgen05.mma.cta_group::2 on a 256 x 256 output tile shared by the
// two CTAs of a thread-block cluster (two SMs of one TPC).
//
// Why: the single-CTA kernel (gemm_sm100.cu) moves (128 + 256) x 64 operand elements per
// 128 x 256 x 64 MMA block, 85 FLOP per byte of shared-memory fill, and measurements put it at the
// L2 -> SM feed limit. In the pair, each CTA loads HALF of each operand (128 rows of A, 128 rows of
// B) and the tensor cores of both SMs read both halves: 131 FLOP per byte filled, with no cluster
// multicast load anywhere (every CTA TMA-loads only its own tiles; the loads carry .cta_group::2
// solely so that their completion bytes are counted on the leader CTA's mbarrier).
//
// Per CTA: 6 stages x (16 KB A-half + 16 KB B-half); TMEM 512 columns = two 128 x 256 fp32
// accumulators (rows 128*rank .. of the pair's tile), so the epilogue of tile i overlaps the main
// loop of tile i+1. Roles per CTA: warp 0 TMA producer, warp 1 TMEM owner (+ MMA issuer in the
// leader CTA only), warps 2-9 epilogue (two per TMEM lane quadrant, one accumulator column half each). Cross-CTA signalling:
//   full[s]   (leader)  <- complete_tx from both CTAs' TMA loads
//   empty[s]  (both)    <- tcgen05.commit.cta_group::2 with a 2-CTA arrive mask
//   tfull[a]  (both)    <- same, after the last k-block of a tile
//   tempty[a] (leader)  <- 8 local + 8 remote (mapa) arrives from the epilogue warps
// Every wait is bounded (status word + abort flag), both CTAs always reach the final cluster barrier.
#include "gemm_common.cuh"
#include <cooperative_groups.h>
#include <cstdlib>

namespace pb {

constexpr int G2_STAGES = 5;
constexpr int G2_HALF_BYTES = 128 * BK * 2;               // 16 KB: 128 rows x 64 bf16
constexpr int G2_STAGE_BYTES = 2 * G2_HALF_BYTES;         // per CTA
constexpr int G2_BN = 256;
constexpr int G2_BOX_BYTES = 128 * 64 * 2;                // one epilogue staging box: 128 rows x 64 bf16, 128B-swizzled
constexpr int G2_EPI_BOXES = 4;
constexpr int G2_SMEM_BYTES = G2_STAGES * G2_STAGE_BYTES + G2_EPI_BOXES * G2_BOX_BYTES + 1024 + 256;

// output-side tensor maps of the staged epilogue (bf16, box = 64 columns x 128 rows)
struct EpiMaps {
    CUtensorMap c;      // C
    CUtensorMap aux;    // SwiGLU: act; dSwiGLU: h13
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes land on an mbarrier that may live in the peer CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void umma2_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on the mbarrier at this shared-memory offset in both CTAs of the pair once all MMAs issued so far retire
__device__ __forceinline__ void umma2_commit_both(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
// One k-block (BK = 64 = four K-steps of 16) of the CTA-pair MMA in a single instruction sequence:
// poll the full-barrier of the NEXT k-block, issue the four MMAs of this one, commit to the stage's
// empty barrier (and to the accumulator-full barrier after the last k-block of a tile), and only then
// consume the poll result. The descriptors of K-steps 1..3 differ from step 0 in the 14-bit start
// address field only (+32 B for a K-major tile, +2048 B for an MN-major one, in 16-byte units).
template <bool A_MN, bool B_MN>
__device__ __forceinline__ bool umma2_kblock(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, bool accumulate,
                                             uint32_t bar_empty, uint32_t bar_tfull, bool last_kb, uint32_t bar_next,
                                             uint32_t parity_next, bool peek) {
    constexpr uint32_t inc_a = A_MN ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
    constexpr uint32_t inc_b = B_MN ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
    uint32_t ready;
    const uint16_t mask = 3;
    asm volatile(
        "{\n\t"
        ".reg .pred P, Q, T, L, K;\n\t"
        ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
        "setp.ne.b32 K, %11, 0;\n\t"
        "setp.ne.b32 P, 0, 0;\n\t"
        "@K mbarrier.try_wait.parity.shared::cta.b64 P, [%9], %10;\n\t"
        "setp.ne.b32 Q, %5, 0;\n\t"
        "setp.eq.b32 T, 0, 0;\n\t"
        "setp.ne.b32 L, %8, 0;\n\t"
        "add.s64 a1, %2, %12;\n\t"
        "add.s64 a2, a1, %12;\n\t"
        "add.s64 a3, a2, %12;\n\t"
        "add.s64 b1, %3, %13;\n\t"
        "add.s64 b2, b1, %13;\n\t"
        "add.s64 b3, b2, %13;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %2, %3, %4, Q;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], a1, b1, %4, T;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], a2, b2, %4, T;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], a3, b3, %4, T;\n\t"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%6], %14;\n\t"
        "@L tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%7], %14;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ready)
        : "r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(uint32_t(accumulate)), "r"(bar_empty), "r"(bar_tfull),
          "r"(uint32_t(last_kb)), "r"(bar_next), "r"(parity_next), "r"(uint32_t(peek)), "l"(uint64_t(inc_a)),
          "l"(uint64_t(inc_b)), "h"(mask)
        : "memory");
    return ready != 0;
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---- all-gather fused into the GEMM (ZeRO-3 parameter gather + first consuming GEMM) ----
// B ([N, K] weights) exists only as per-rank row shards in symmetric memory. The epilogue warps of
// every CTA, idle until the first accumulator completes, pull the remote rows with plain P2P loads
// into this GPU's full-size B buffer in sub-units of GATHER_ROWS rows and bump a per-n-block counter;
// the TMA producers wait (bounded) on the counter of the n-block they are about to load. The gather
// of later n-blocks therefore overlaps the math of earlier tiles, and every remote byte crosses
// NVLink exactly once. No multicast, no library call on peer memory.
constexpr int GATHER_ROWS = 32;
constexpr int GATHER_MAX_RANKS = 16;
constexpr int GATHER_MAX_PARTS = 4;
struct GatherParams {
    int world, rank;
    // B is the row-wise concatenation of n_parts matrices (e.g. wq | wk | wv), each row-sharded over the ranks on its own:
    // rows [part_begin[p], part_begin[p + 1]) belong to part p, rank r owns rows_per_rank[p] consecutive rows of it starting
    // at r * rows_per_rank[p], and keeps them at shard[r] + part_off[p] (row pitch ld)
    const __nv_bfloat16* shard[GATHER_MAX_RANKS];
    int n_parts;
    int part_begin[GATHER_MAX_PARTS + 1];
    int rows_per_rank[GATHER_MAX_PARTS];
    long long part_off[GATHER_MAX_PARTS];
    int unit_rot;                                   // gather order: sub-unit (i + unit_rot) mod n_units is the i-th to be fetched
    __nv_bfloat16* full;                            // local [N, ld] buffer the TMA map of B points at
    long long ld;
    int* counters;                                  // [ceil(N/256)] monotonically increasing sub-unit counts
    int target;                                     // counter value that means "n-block complete" for this launch
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

template <bool A_MN, bool B_MN, bool GATHER, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(320, 1)
gemm_bf16_tcgen05_pair(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ EpiMaps em, const GemmParams p, const GatherParams g) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t s_epi = smem_base + G2_STAGES * G2_STAGE_BYTES;      // [G2_EPI_BOXES] staging boxes
    uint8_t* g_epi = smem_gen + G2_STAGES * G2_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + G2_STAGES * G2_STAGE_BYTES + G2_EPI_BOXES * G2_BOX_BYTES);
    const uint32_t bar_full = smem_u32(bars);                     // [STAGES]   used in the leader
    const uint32_t bar_empty = bar_full + 8 * G2_STAGES;          // [STAGES]   each CTA
    const uint32_t bar_tfull = bar_empty + 8 * G2_STAGES;         // [2]        each CTA
    const uint32_t bar_tempty = bar_tfull + 16;                   // [2]        used in the leader
    const uint32_t bar_eload = bar_tempty + 16;                   // [2]        staged epilogue: input boxes have landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * G2_STAGES + 6);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < G2_STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, 16);      // 8 epilogue warps x 2 CTAs
            mbar_init(bar_eload + 8 * a, 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc2(smem_u32(tmem_slot), 512);
        tmem_relinquish2();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the peer's barriers exist before anything can signal them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int num_kb = (p.K + BK - 1) / BK;
    // the leader's copies of the barriers this CTA signals remotely
    const uint32_t lead_full = mapa_shared(bar_full, 0);
    const uint32_t lead_tempty = mapa_shared(bar_tempty, 0);

    if (warp == 0) {
        // ------------------------- TMA producer (both CTAs) -------------------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        unsigned long long gathered_mask = 0ull;           // all-gather GEMM: n-blocks already seen complete
        (void)gathered_mask;
        for (int item = pair; item < p.num_items && ok; item += n_pairs) {
            const int tile = item % p.num_tiles, slice = item / p.num_tiles;
            const int kb0 = slice * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
            int tm, tn;
            gemm_tile_mn(p, tile, tm, tn);
            const int m0 = tm * 256 + int(rank) * 128;     // my half of the A rows
            // my half of the B rows; with the SwiGLU epilogue the halves are the gate rows and the matching up rows
            const int n0 = EPI == GEMM_EPI_SWIGLU ? tn * 128 + int(rank) * p.epi_i0 : tn * G2_BN + int(rank) * 128;
            if constexpr (GATHER) {
                // wait until every row of this n-block has landed in the local B buffer; an n-block seen complete once is
                // not polled again (the counters only grow)
                const bool known = tn < 64 && ((gathered_mask >> tn) & 1ull);
                if (!known) {
                    const int* ctr = g.counters + tn;
                    const uint64_t t0 = globaltimer_ns();
                    while (ok && ld_acquire_gpu(ctr) < g.target) {
                        if (*abort_flag) ok = false;
                        else if (globaltimer_ns() - t0 > PB_WAIT_BUDGET_NS) {
                            *abort_flag = 1;
                            if (p.status) atomicCAS(p.status, 0, PB_ERR_TIMEOUT_PEER | (int(blockIdx.x) << 8));
                            ok = false;
                        }
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    fence_proxy_async_global();      // generic-proxy stores of the gather -> async-proxy (TMA) reads
                    if (tn < 64) gathered_mask |= 1ull << tn;
                }
            }
            for (int kb = kb0; kb < kb1; ++kb) {
                ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, PB_ERR_TIMEOUT_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t sa = smem_base + stage * G2_STAGE_BYTES;
                    const uint32_t sb = sa + G2_HALF_BYTES;
                    const uint32_t fb = lead_full + 8 * stage;
                    if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * G2_STAGE_BYTES);   // bytes of both CTAs
                    const int k0 = kb * BK;
                    if constexpr (!A_MN) {
                        tma_load_2d_pair(sa, &tmA, fb, k0, m0);
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tmA, fb, m0 + 64 * j, k0);
                    }
                    if constexpr (!B_MN) {
                        tma_load_2d_pair(sb, &tmB, fb, k0, n0);
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j) tma_load_2d_pair(sb + j * (BK * 128), &tmB, fb, n0 + 64 * j, k0);
                    }
                }
                __syncwarp();
                if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
            }
        }
        if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(10000);
    } else if (warp == 1) {
        // ------------------------- MMA issuer (leader CTA only) -------------------------
        // One thread runs the whole loop. While the four MMAs of a k-block are being issued, the
        // full-barrier of the next k-block is already being polled (its latency is hidden behind the
        // issue instead of being paid between k-blocks).
        if (rank == 0 && lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(256, G2_BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
            int stage = 0, local = 0;
            uint32_t phase = 0;
            bool ok = true, ready = false;
            for (int item = pair; item < p.num_items && ok; item += n_pairs, ++local) {
                const int slice = item / p.num_tiles;
                const int kb0 = slice * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
                const bool last_item = item + n_pairs >= p.num_items;
                const int acc = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                ok = mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                const uint32_t d_tmem = tmem_base + acc * G2_BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!ready) {
                        ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, PB_ERR_TIMEOUT_FULL);
                        if (!ok) break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_base + stage * G2_STAGE_BYTES;
                    const uint32_t sb = sa + G2_HALF_BYTES;
                    const uint64_t da = A_MN ? umma_smem_desc(sa, BK * 128, 1024) : umma_smem_desc(sa, 16, 1024);
                    const uint64_t db = B_MN ? umma_smem_desc(sb, BK * 128, 1024) : umma_smem_desc(sb, 16, 1024);
                    const int nstage = stage + 1 == G2_STAGES ? 0 : stage + 1;
                    const uint32_t nphase = nstage == 0 ? phase ^ 1 : phase;
                    ready = umma2_kblock<A_MN, B_MN>(d_tmem, da, db, idesc, kb != kb0, bar_empty + 8 * stage,
                                                     bar_tfull + 8 * acc, kb == kb1 - 1, bar_full + 8 * nstage, nphase,
                                                     !(last_item && kb == kb1 - 1));
                    stage = nstage;
                    phase = nphase;
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------- epilogue (warps 2..9, both CTAs) -------------------------
        // warp w reads TMEM lane quadrant w & 3 (a hardware rule) and column half (w - 2) >> 2 of the accumulator
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row_in_half = quad * 32 + lane;
        if constexpr (GATHER) {
            const int et = threadIdx.x - 64;                       // 0..255 within the eight epilogue warps
            const int n_units = (p.N + GATHER_ROWS - 1) / GATHER_ROWS;
            const int vec_per_row = p.K / 8;                       // 16-byte vectors per row (K % 8 == 0)
            for (int u0 = blockIdx.x; u0 < n_units; u0 += gridDim.x) {
                // rotated by rank: the n-blocks the tiles start with come first, and the ranks do not all pull from one peer
                const int u = (u0 + g.unit_rot) % n_units;
                const int r0 = u * GATHER_ROWS, r1 = min(p.N, r0 + GATHER_ROWS);
                int part = 0;
                while (part + 1 < g.n_parts && r0 >= g.part_begin[part + 1]) ++part;
                const int local = r0 - g.part_begin[part];         // GATHER_ROWS divides every part and every rows_per_rank
                const int owner = local / g.rows_per_rank[part];
                if (owner != g.rank) {
                    const __nv_bfloat16* src = g.shard[owner] + g.part_off[part] + (long long)(local - owner * g.rows_per_rank[part]) * g.ld;
                    __nv_bfloat16* dst = g.full + (long long)r0 * g.ld;
                    const int total = (r1 - r0) * vec_per_row;
                    for (int i = et; i < total; i += 256 * 4) {    // 4 independent 16-byte peer loads in flight per thread
                        uint4 v[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int j = i + k * 256;
                            if (j < total) v[k] = *reinterpret_cast<const uint4*>(src + (long long)(j / vec_per_row) * g.ld + (j % vec_per_row) * 8);
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int j = i + k * 256;
                            if (j < total) *reinterpret_cast<uint4*>(dst + (long long)(j / vec_per_row) * g.ld + (j % vec_per_row) * 8) = v[k];
                        }
                    }
                }
                __threadfence();
                asm volatile("bar.sync 1, 256;" ::: "memory");      // the eight epilogue warps only
                if (et == 0) {
                    fence_proxy_async_global();
                    asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(g.counters + r0 / G2_BN) : "memory");
                }
            }
        }
        // The bf16 epilogues go through shared memory: every thread writes its row piece of a
        // 128-row x 64-column box (128B-swizzled), one thread hands the box to TMA. Global memory then sees
        // whole 128-byte rows instead of 64-byte pieces 32 rows apart; the fused SwiGLU backward also
        // fetches its inputs that way, one block ahead. fp32 outputs and residual adds use direct stores.
        const int et = threadIdx.x - 64;                           // 0..255 within the eight epilogue warps
        const bool staged = EPI == GEMM_EPI_SWIGLU || EPI == GEMM_EPI_DSWIGLU || EPI == GEMM_EPI_ROWDOT || EPI == GEMM_EPI_ADD || p.staged;
        auto epi_sync = [] { asm volatile("bar.sync 2, 256;" ::: "memory"); };
        // this thread's 64-byte piece (32 bf16 = chunks ch0..ch0+3 of 16 bytes) of row r in a staging box
        auto box_off = [&](int box, int ch) { return box * G2_BOX_BYTES + row_in_half * 128 + (((ch) ^ (row_in_half & 7)) << 4); };
        int local = 0;
        uint32_t rounds = 0;                                       // staged rounds done (buffer / phase bookkeeping)
        bool ok = true;
        if constexpr (EPI == GEMM_EPI_DSWIGLU) {
            // gate | up of the first block of the first tile
            if (et == 0 && pair < p.num_items) {
                int tm, tn;
                gemm_tile_mn(p, pair, tm, tn);
                const int m0 = tm * 256 + int(rank) * 128, n0 = tn * G2_BN;
                mbar_expect_tx(bar_eload, 2 * G2_BOX_BYTES);
                tma_load_2d(s_epi, &em.aux, bar_eload, n0, m0);
                tma_load_2d(s_epi + G2_BOX_BYTES, &em.aux, bar_eload, p.epi_i0 + n0, m0);
            }
        }
        if constexpr (EPI == GEMM_EPI_ROWDOT || EPI == GEMM_EPI_ADD) {
            // the two 64-column boxes of the other matrix for the first round of the first tile
            if (et == 0 && pair < p.num_items) {
                int tm, tn;
                gemm_tile_mn(p, pair, tm, tn);
                const int m0 = tm * 256 + int(rank) * 128, n0 = tn * G2_BN;
                mbar_expect_tx(bar_eload, 2 * G2_BOX_BYTES);
                tma_load_2d(s_epi, &em.aux, bar_eload, n0, m0);
                tma_load_2d(s_epi + G2_BOX_BYTES, &em.aux, bar_eload, n0 + 64, m0);
            }
        }
        for (int item = pair; item < p.num_items && ok; item += n_pairs, ++local) {
            const int tile = item % p.num_tiles, slice = item / p.num_tiles;
            const int acc = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            int tm, tn;
            gemm_tile_mn(p, tile, tm, tn);
            const int m0 = tm * 256 + int(rank) * 128;
            const int n0 = tn * G2_BN;
            ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = m0 + row_in_half;
            const uint32_t t_row = tmem_base + acc * G2_BN + (uint32_t(quad * 32) << 16);
            auto release_acc = [&] {   // this warp has read all it needs of the accumulator
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(lead_tempty + 8 * acc);
            };
            if constexpr (EPI == GEMM_EPI_SWIGLU) {
                // two rounds of 64 features: boxes 0, 1, 2 = gate, up, act; this warp does 32 of the 64 columns
                const int F = p.epi_i0;
                const int j0 = tn * 128;
#pragma unroll 1
                for (int rnd = 0; rnd < 2; ++rnd) {
                    uint32_t vg[32], vu[32];
                    tmem_ld32(t_row + rnd * 64 + half * 32, vg);          // gate: accumulator columns 0..127
                    tmem_ld32(t_row + 128 + rnd * 64 + half * 32, vu);    // up:   accumulator columns 128..255
                    if (et == 0) tma_store_wait_read<0>();                // the boxes of the previous round have been read
                    epi_sync();
                    tmem_ld_wait();
                    if (rnd == 1) release_acc();
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint32_t og[4], ou[4], oa[4];
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            const float g0 = __uint_as_float(vg[8 * q + 2 * t]), g1 = __uint_as_float(vg[8 * q + 2 * t + 1]);
                            const float u0 = __uint_as_float(vu[8 * q + 2 * t]), u1 = __uint_as_float(vu[8 * q + 2 * t + 1]);
                            og[t] = pack_bf16x2(g0, g1);
                            ou[t] = pack_bf16x2(u0, u1);
                            oa[t] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
                        }
                        *reinterpret_cast<uint4*>(g_epi + box_off(0, half * 4 + q)) = make_uint4(og[0], og[1], og[2], og[3]);
                        *reinterpret_cast<uint4*>(g_epi + box_off(1, half * 4 + q)) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
                        *reinterpret_cast<uint4*>(g_epi + box_off(2, half * 4 + q)) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
                    }
                    fence_proxy_async_smem();
                    epi_sync();
                    if (et == 0) {
                        tma_store_2d(&em.c, s_epi, j0 + rnd * 64, m0);
                        tma_store_2d(&em.c, s_epi + G2_BOX_BYTES, F + j0 + rnd * 64, m0);
                        tma_store_2d(&em.aux, s_epi + 2 * G2_BOX_BYTES, j0 + rnd * 64, m0);
                        tma_store_commit();
                    }
                }
            } else if constexpr (EPI == GEMM_EPI_DSWIGLU) {
                // four rounds of 64 columns of d(act); buffer b = boxes 2b (gate) and 2b+1 (up), rewritten in place
                const int F = p.epi_i0;
#pragma unroll 1
                for (int rnd = 0; rnd < 4; ++rnd, ++rounds) {
                    const int buf = rounds & 1;
                    uint32_t v[32];
                    tmem_ld32(t_row + rnd * 64 + half * 32, v);
                    if (et == 0) {
                        // fetch the next block (of this tile or of the next one) into the other buffer
                        int nt = tile, nr = rnd + 1;
                        if (nr == 4) { nr = 0; nt += n_pairs; }
                        if (nt < p.num_tiles) {
                            int ntm, ntn;
                            gemm_tile_mn(p, nt, ntm, ntn);
                            const int nm0 = ntm * 256 + int(rank) * 128, nn0 = ntn * G2_BN + nr * 64;
                            tma_store_wait_read<0>();      // the stores that last used that buffer have read it
                            if (nn0 < p.N) {
                                mbar_expect_tx(bar_eload + 8 * (buf ^ 1), 2 * G2_BOX_BYTES);
                                tma_load_2d(s_epi + (2 * (buf ^ 1)) * G2_BOX_BYTES, &em.aux, bar_eload + 8 * (buf ^ 1), nn0, nm0);
                                tma_load_2d(s_epi + (2 * (buf ^ 1) + 1) * G2_BOX_BYTES, &em.aux, bar_eload + 8 * (buf ^ 1), F + nn0, nm0);
                            } else {
                                mbar_arrive(bar_eload + 8 * (buf ^ 1));   // block past N: nothing to fetch, keep the phases in step
                            }
                        }
                    }
                    ok = mbar_wait(bar_eload + 8 * buf, (rounds >> 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_MISC);
                    ok = __all_sync(0xffffffffu, ok);
                    tmem_ld_wait();
                    if (rnd == 3) release_acc();
                    if (!ok) break;
                    const bool live = n0 + rnd * 64 < p.N;
                    if (live) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint4* pg = reinterpret_cast<uint4*>(g_epi + box_off(2 * buf, half * 4 + q));
                            uint4* pu = reinterpret_cast<uint4*>(g_epi + box_off(2 * buf + 1, half * 4 + q));
                            const uint4 cg = *pg, cu = *pu;
                            const uint32_t gw[4] = {cg.x, cg.y, cg.z, cg.w};
                            const uint32_t uw[4] = {cu.x, cu.y, cu.z, cu.w};
                            uint32_t og[4], ou[4];
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                const float2 g2 = unpack_bf16x2(gw[t]), u2 = unpack_bf16x2(uw[t]);
                                const float d0 = __uint_as_float(v[8 * q + 2 * t]), d1 = __uint_as_float(v[8 * q + 2 * t + 1]);
                                const float s0 = 1.f / (1.f + __expf(-g2.x)), s1 = 1.f / (1.f + __expf(-g2.y));
                                og[t] = pack_bf16x2(d0 * u2.x * s0 * (1.f + g2.x * (1.f - s0)), d1 * u2.y * s1 * (1.f + g2.y * (1.f - s1)));
                                ou[t] = pack_bf16x2(d0 * g2.x * s0, d1 * g2.y * s1);
                            }
                            *pg = make_uint4(og[0], og[1], og[2], og[3]);
                            *pu = make_uint4(ou[0], ou[1], ou[2], ou[3]);
                        }
                    }
                    fence_proxy_async_smem();
                    epi_sync();
                    if (et == 0 && live) {
                        tma_store_2d(&em.aux, s_epi + (2 * buf) * G2_BOX_BYTES, n0 + rnd * 64, m0);
                        tma_store_2d(&em.aux, s_epi + (2 * buf + 1) * G2_BOX_BYTES, F + n0 + rnd * 64, m0);
                        tma_store_commit();
                    }
                }
            } else if constexpr (EPI == GEMM_EPI_ROWDOT || EPI == GEMM_EPI_ADD) {
                // two rounds of 128 columns; buffer b = boxes 2b, 2b+1 arrive holding the other matrix and leave
                // holding C; this warp owns box `half` of the round = the 64 columns of one head of its row
#pragma unroll 1
                for (int rnd = 0; rnd < 2; ++rnd, ++rounds) {
                    const int buf = rounds & 1;
                    uint32_t v0[32], v1[32];
                    tmem_ld32(t_row + rnd * 128 + half * 64, v0);
                    tmem_ld32(t_row + rnd * 128 + half * 64 + 32, v1);
                    if (et == 0) {
                        int nt = tile, nr = rnd + 1;
                        if (nr == 2) { nr = 0; nt += n_pairs; }
                        if (nt < p.num_tiles) {
                            int ntm, ntn;
                            gemm_tile_mn(p, nt, ntm, ntn);
                            const int nm0 = ntm * 256 + int(rank) * 128, nn0 = ntn * G2_BN + nr * 128;
                            tma_store_wait_read<0>();      // the stores that last used that buffer have read it
                            mbar_expect_tx(bar_eload + 8 * (buf ^ 1), 2 * G2_BOX_BYTES);   // columns past N arrive as zeros
                            tma_load_2d(s_epi + (2 * (buf ^ 1)) * G2_BOX_BYTES, &em.aux, bar_eload + 8 * (buf ^ 1), nn0, nm0);
                            tma_load_2d(s_epi + (2 * (buf ^ 1) + 1) * G2_BOX_BYTES, &em.aux, bar_eload + 8 * (buf ^ 1), nn0 + 64, nm0);
                        }
                    }
                    ok = mbar_wait(bar_eload + 8 * buf, (rounds >> 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_MISC);
                    ok = __all_sync(0xffffffffu, ok);
                    tmem_ld_wait();
                    if (rnd == 1) release_acc();
                    if (!ok) break;
                    const int cb = n0 + rnd * 128 + half * 64;
                    float dot = 0.f;
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        uint32_t (&v)[32] = hh ? v1 : v0;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint4* px = reinterpret_cast<uint4*>(g_epi + box_off(2 * buf + half, hh * 4 + q));
                            const uint4 x = *px;
                            const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
                            uint32_t o[4];
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                const float2 x2 = unpack_bf16x2(xw[t]);
                                const float c0 = __uint_as_float(v[8 * q + 2 * t]), c1 = __uint_as_float(v[8 * q + 2 * t + 1]);
                                if constexpr (EPI == GEMM_EPI_ADD) {
                                    o[t] = pack_bf16x2(c0 + x2.x, c1 + x2.y);
                                } else {
                                    dot += c0 * x2.x + c1 * x2.y;
                                    o[t] = pack_bf16x2(c0, c1);
                                }
                            }
                            *px = make_uint4(o[0], o[1], o[2], o[3]);
                        }
                    }
                    if (EPI == GEMM_EPI_ROWDOT && row < p.M && cb < p.N) reinterpret_cast<float*>(p.aux2)[(long long)(cb / 64) * p.M + row] = dot;
                    fence_proxy_async_smem();
                    epi_sync();
                    if (et == 0) {
#pragma unroll
                        for (int h2 = 0; h2 < 2; ++h2)
                            if (n0 + rnd * 128 + h2 * 64 < p.N)
                                tma_store_2d(&em.c, s_epi + (2 * buf + h2) * G2_BOX_BYTES, n0 + rnd * 128 + h2 * 64, m0);
                        tma_store_commit();
                    }
                }
            } else if (staged) {
                // two rounds of 128 columns; buffer b = boxes 2b, 2b+1; this warp fills box `half` of the round
                constexpr bool rope = EPI == GEMM_EPI_ROPE;
                const float* cs_row = rope ? reinterpret_cast<const float*>(p.aux) + (long long)(row % p.epi_i0) * p.epi_i2 : nullptr;
#pragma unroll 1
                for (int rnd = 0; rnd < 2; ++rnd, ++rounds) {
                    const int buf = rounds & 1;
                    const int cb = n0 + rnd * 128 + half * 64;             // first column of this warp's box
                    uint32_t v0[32], v1[32];
                    tmem_ld32(t_row + rnd * 128 + half * 64, v0);
                    tmem_ld32(t_row + rnd * 128 + half * 64 + 32, v1);
                    float4 cs[16];
                    const bool rot = rope && cb < p.epi_i1;
                    if (rot) {
#pragma unroll
                        for (int q = 0; q < 16; ++q) cs[q] = *reinterpret_cast<const float4*>(cs_row + (cb % p.epi_i2) + 4 * q);
                    }
                    if (et == 0) tma_store_wait_read<1>();                 // the stores that last used this buffer have read it
                    epi_sync();
                    tmem_ld_wait();
                    if (rnd == 1) release_acc();
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        uint32_t (&v)[32] = hh ? v1 : v0;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t o[4];
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                float x = __uint_as_float(v[8 * q + 2 * t]), y = __uint_as_float(v[8 * q + 2 * t + 1]);
                                if (rot) {   // (even, odd) pair idx within the 64-column box: hh*16 + 4q + t
                                    const float4 c4 = cs[(hh * 16 + 4 * q + t) >> 1];
                                    const float co = (t & 1) ? c4.z : c4.x, si = (t & 1) ? c4.w : c4.y;
                                    const float xr = x * co - y * si;
                                    y = x * si + y * co;
                                    x = xr;
                                }
                                o[t] = pack_bf16x2(x, y);
                            }
                            *reinterpret_cast<uint4*>(g_epi + box_off(2 * buf + half, hh * 4 + q)) = make_uint4(o[0], o[1], o[2], o[3]);
                        }
                    }
                    fence_proxy_async_smem();
                    epi_sync();
                    if (et == 0) {
#pragma unroll
                        for (int h2 = 0; h2 < 2; ++h2)
                            if (n0 + rnd * 128 + h2 * 64 < p.N)
                                tma_store_2d(&em.c, s_epi + (2 * buf + h2) * G2_BOX_BYTES, n0 + rnd * 128 + h2 * 64, m0);
                        tma_store_commit();
                    }
                }
            } else {
                const int cbeg = half * 128;
                GemmParams ps = p;
                if (slice) ps.C = reinterpret_cast<float*>(p.C) + slice * p.split_stride;   // split-K partials are fp32
#pragma unroll 1
                for (int c = cbeg; c < cbeg + 128; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(t_row + c, v);
                    tmem_ld_wait();
                    gemm_store_chunk(ps, v, row, n0 + c);
                }
                release_acc();
            }
        }
        if (et == 0) tma_store_wait<0>();   // every staged store of this CTA has landed
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // nobody leaves while the pair may still touch its memory
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, 512);
    }
}

// Rows of tiles per band of the tile numbering (gemm_tile_mn). Row-major numbering reads A once and B once per wave of
// CTA pairs, which is free while B stays in L2; a B operand that does not fit there (48 MB and more: the 10B model's
// w13 and head, the 150M model's head) would be streamed from HBM tiles_m / (rows per wave) times, so such products
// use bands of 16 rows: [8192 x 128256 x 4096] 8.22 -> 5.81 ms, [8192 x 28672 x 4096] 1.61 -> 1.25 ms, while products
// with a small B, or with so few tile columns that a wave spans several tile rows anyway, lose 1-2 % to banding and
// keep the row-major order. PRIME_B200_GEMM_GROUP_M overrides (measurements).
static int tile_band_rows(int tiles_m, int tiles_n, long long b_bytes) {
    static const int forced = [] { const char* e = getenv("PRIME_B200_GEMM_GROUP_M"); return e ? atoi(e) : 0; }();
    if (forced > 0) return forced;
    return (b_bytes >= (48ll << 20) && tiles_n >= 32 && tiles_m >= 8) ? 16 : 1;
}

template <bool A_MN, bool B_MN, bool GATHER = false, int EPI = GEMM_EPI_NONE>
static int launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams p, int max_ctas, cudaStream_t st,
                            const GatherParams& g = GatherParams{}, const EpiMaps& em = EpiMaps{}) {
    auto kern = gemm_bf16_tcgen05_pair<A_MN, B_MN, GATHER, EPI>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_BYTES) != cudaSuccess) return -20;
        configured = true;
    }
    const int tiles_m = (p.M + 255) / 256;
    p.tiles_n = EPI == GEMM_EPI_SWIGLU ? p.epi_i0 / 128 : (p.N + G2_BN - 1) / G2_BN;
    p.num_tiles = tiles_m * p.tiles_n;
    p.tiles_m = tiles_m;
    // with the gather fused in, tiles are numbered in bands of 8 tile rows starting at the n-block the gather fetches first: the
    // first wave then waits for part of B, not for all of it, while a band's A rows still stay in L2 across its n-blocks
    // (measured at M32768 N4096 K1024, 2 GPUs: bands of 1 or 8 rows 241 us, 16 rows 247 us, whole columns 278 us)
    static const int ag_group = [] { const char* e = getenv("PRIME_B200_AG_GROUP_M"); return e ? atoi(e) : 0; }();
    p.group_m = GATHER ? (ag_group > 0 ? (ag_group < tiles_m ? ag_group : tiles_m) : (tiles_m < 8 ? tiles_m : 8))
                       : tile_band_rows(tiles_m, p.tiles_n, 2ll * p.N * p.K);
    p.tn_rot = GATHER ? (g.unit_rot / (G2_BN / GATHER_ROWS)) % p.tiles_n : 0;
    if (p.num_items <= 0) {   // no split-K requested
        p.num_items = p.num_tiles;
        p.kb_per_split = (p.K + BK - 1) / BK;
    } else {
        p.num_items *= p.num_tiles;   // the caller passed the number of K slices
    }
    int ctas = sm_count() & ~1;
    if (max_ctas > 0 && ctas > (max_ctas & ~1)) ctas = max_ctas & ~1;
    if (ctas > 2 * p.num_items) ctas = 2 * p.num_items;
    if (ctas < 2) ctas = 2;
    kern<<<ctas, 320, G2_SMEM_BYTES, st>>>(tmA, tmB, em, p, g);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

}  // namespace pb

extern "C" int pb_gemm_bf16_pair_epi(const void* A, const void* B, void* C, const void* R, int M, int N, int K, long long lda,
                                     long long ldb, long long ldc, long long ldr, int a_mn, int b_mn, int out_fp32, int max_ctas,
                                     int epi, int epi_i0, int epi_i1, int epi_i2, void* aux, long long ldaux, void* aux2,
                                     int* status, void* stream);

// Same contract as pb_gemm_bf16; requires nothing more of the operands. Tile 256 x 256 per CTA pair.
extern "C" int pb_gemm_bf16_pair(const void* A, const void* B, void* C, const void* R, int M, int N, int K, long long lda,
                                 long long ldb, long long ldc, long long ldr, int a_mn, int b_mn, int out_fp32, int max_ctas,
                                 int* status, void* stream) {
    return pb_gemm_bf16_pair_epi(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, a_mn, b_mn, out_fp32, max_ctas, 0, 0, 0, 0, nullptr, 0,
                                 nullptr, status, stream);
}

// pb_gemm_bf16_pair with one of the fused epilogues described next to GEMM_EPI_* (bf16 output only):
//   epi 1 (SwiGLU)  : B = [w1; w3] K-major, N = 2F, epi_i0 = F (multiple of 128), C = h13, aux = act, ldaux its pitch
//   epi 2 (RoPE)    : epi_i0 = T, epi_i1 = number of leading columns to rotate, epi_i2 = head size, aux = fp32 table
//   epi 3 (dSwiGLU) : N = F = epi_i0, aux = h13 (read gate | up, written d gate | d up), C unused
//   epi 4 (row dot) : aux = bf16 [M, N] with pitch ldaux, epi_i0 = 64 columns per group, aux2 = fp32 [N / 64, M]
//   epi 5 (add)     : aux = bf16 [M, N] addend with pitch ldaux (may be C)
extern "C" int pb_gemm_bf16_pair_epi(const void* A, const void* B, void* C, const void* R, int M, int N, int K, long long lda,
                                     long long ldb, long long ldc, long long ldr, int a_mn, int b_mn, int out_fp32, int max_ctas,
                                     int epi, int epi_i0, int epi_i1, int epi_i2, void* aux, long long ldaux, void* aux2,
                                     int* status, void* stream) {
    using namespace pb;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (epi != GEMM_EPI_NONE) {
        if (out_fp32 || R || !aux || (reinterpret_cast<uintptr_t>(aux) & 15)) return -4;
        if (epi == GEMM_EPI_SWIGLU && (a_mn || b_mn || epi_i0 % 128 || N != 2 * epi_i0 || ldaux % 8)) return -4;
        if (epi == GEMM_EPI_ROPE && (a_mn || b_mn || epi_i0 <= 0 || epi_i2 % 64 || epi_i1 % 64 || epi_i1 > N)) return -4;
        if (epi == GEMM_EPI_DSWIGLU && (a_mn || !b_mn || N != epi_i0 || epi_i0 % 64 || ldaux % 8)) return -4;
        if (epi == GEMM_EPI_ROWDOT && (a_mn || epi_i0 != 64 || ldaux % 8 || !aux2)) return -4;
        if (epi == GEMM_EPI_ADD && (ldaux % 8)) return -4;
        if (epi < 0 || epi > GEMM_EPI_ADD) return -4;
    }
    if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -1;
    const int vec = out_fp32 ? 4 : 8;
    if ((ldc % vec) || (R && (ldr % vec)) || (reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(R) & 15)) return -2;
    CUtensorMap tmA, tmB;
    int rc;
    if (!a_mn) rc = make_tmap_bf16_2d(&tmA, A, K, M, lda, BK, 128);
    else       rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, 64, BK);
    if (rc) return rc;
    if (!b_mn) rc = make_tmap_bf16_2d(&tmB, B, K, N, ldb, BK, 128);
    else       rc = make_tmap_bf16_2d(&tmB, B, N, K, ldb, 64, BK);
    if (rc) return rc;
    GemmParams p{};
    p.M = M; p.N = N; p.K = K; p.C = C; p.R = R; p.ldc = ldc; p.ldr = ldr; p.out_fp32 = out_fp32; p.status = status;
    p.epi = epi; p.epi_i0 = epi_i0; p.epi_i1 = epi_i1; p.epi_i2 = epi_i2; p.aux = aux; p.ldaux = ldaux; p.aux2 = aux2;
    // bf16 tiles without a residual leave through shared memory + TMA stores
    p.staged = (!out_fp32 && !R && epi != GEMM_EPI_DSWIGLU) ? 1 : 0;
    EpiMaps em{};
    if (p.staged) {
        rc = make_tmap_bf16_2d(&em.c, C, N, M, ldc, 64, 128);
        if (rc) return rc;
    }
    if (epi == GEMM_EPI_SWIGLU) rc = make_tmap_bf16_2d(&em.aux, aux, epi_i0, M, ldaux, 64, 128);
    if (epi == GEMM_EPI_DSWIGLU) rc = make_tmap_bf16_2d(&em.aux, aux, 2 * uint64_t(epi_i0), M, ldaux, 64, 128);
    if (epi == GEMM_EPI_ROWDOT || epi == GEMM_EPI_ADD) rc = make_tmap_bf16_2d(&em.aux, aux, N, M, ldaux, 64, 128);
    if (rc) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const GatherParams ng{};
    if (epi == GEMM_EPI_SWIGLU) return launch_gemm_pair<false, false, false, GEMM_EPI_SWIGLU>(tmA, tmB, p, max_ctas, st, ng, em);
    if (epi == GEMM_EPI_ROPE) return launch_gemm_pair<false, false, false, GEMM_EPI_ROPE>(tmA, tmB, p, max_ctas, st, ng, em);
    if (epi == GEMM_EPI_DSWIGLU) return launch_gemm_pair<false, true, false, GEMM_EPI_DSWIGLU>(tmA, tmB, p, max_ctas, st, ng, em);
    if (epi == GEMM_EPI_ROWDOT && b_mn) return launch_gemm_pair<false, true, false, GEMM_EPI_ROWDOT>(tmA, tmB, p, max_ctas, st, ng, em);
    if (epi == GEMM_EPI_ROWDOT) return launch_gemm_pair<false, false, false, GEMM_EPI_ROWDOT>(tmA, tmB, p, max_ctas, st, ng, em);
    if (epi == GEMM_EPI_ADD) {
        if (!a_mn && !b_mn) return launch_gemm_pair<false, false, false, GEMM_EPI_ADD>(tmA, tmB, p, max_ctas, st, ng, em);
        if (!a_mn && b_mn)  return launch_gemm_pair<false, true, false, GEMM_EPI_ADD>(tmA, tmB, p, max_ctas, st, ng, em);
        if (a_mn && !b_mn)  return launch_gemm_pair<true, false, false, GEMM_EPI_ADD>(tmA, tmB, p, max_ctas, st, ng, em);
        return launch_gemm_pair<true, true, false, GEMM_EPI_ADD>(tmA, tmB, p, max_ctas, st, ng, em);
    }
    if (!a_mn && !b_mn) return launch_gemm_pair<false, false>(tmA, tmB, p, max_ctas, st, ng, em);
    if (!a_mn && b_mn)  return launch_gemm_pair<false, true>(tmA, tmB, p, max_ctas, st, ng, em);
    if (a_mn && !b_mn)  return launch_gemm_pair<true, false>(tmA, tmB, p, max_ctas, st, ng, em);
    return launch_gemm_pair<true, true>(tmA, tmB, p, max_ctas, st, ng, em);
}

// All-gather fused GEMM: C[M,N] = A[M,K] * B[N,K]^T (+R) where B is row-sharded over `world` ranks.
//   shards[r]   : base of rank r's shard region (peer pointer); part p of B (part_rows[p] rows, part_rows_per_rank[p] of them
//                 per rank) sits at shards[r] + part_off[p] elements, row pitch ldb
//   b_full      : this GPU's [N, ldb] buffer; its own rows must already be in place, the rest is filled here
//   counters    : int[ceil(N/256)], zeroed once by the caller; `call_index` (1, 2, ...) = number of gathers
//                 run on these counters including this one (they only grow, so no reset race exists)
// The caller must order this launch after every rank has published its shard (e.g. SymmComm.barrier()).
// Part sizes and rows per rank must be multiples of 32.
extern "C" int pb_gemm_bf16_allgather_parts(const void* A, void* const* shards, void* b_full, void* C, const void* R, int M, int N, int K,
                                            long long lda, long long ldb, long long ldc, long long ldr, int a_mn, int out_fp32, int world,
                                            int rank, int n_parts, const int* part_rows, const int* part_rows_per_rank,
                                            const long long* part_off, int* counters, int call_index, int max_ctas, int* status,
                                            void* stream) {
    using namespace pb;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (world > GATHER_MAX_RANKS || n_parts < 1 || n_parts > GATHER_MAX_PARTS || (K % 8)) return -1;
    if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(b_full) & 15)) return -1;
    const int vec = out_fp32 ? 4 : 8;
    if ((ldc % vec) || (R && (ldr % vec)) || (reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(R) & 15)) return -2;
    CUtensorMap tmA, tmB;
    int rc = a_mn ? make_tmap_bf16_2d(&tmA, A, M, K, lda, 64, BK) : make_tmap_bf16_2d(&tmA, A, K, M, lda, BK, 128);
    if (rc) return rc;
    rc = make_tmap_bf16_2d(&tmB, b_full, K, N, ldb, BK, 128);
    if (rc) return rc;
    GemmParams p{};
    p.M = M; p.N = N; p.K = K; p.C = C; p.R = R; p.ldc = ldc; p.ldr = ldr; p.out_fp32 = out_fp32; p.status = status;
    GatherParams g{};
    g.world = world; g.rank = rank; g.full = reinterpret_cast<__nv_bfloat16*>(b_full); g.ld = ldb;
    g.n_parts = n_parts;
    int rows = 0;
    for (int i = 0; i < n_parts; ++i) {
        if ((part_rows[i] % GATHER_ROWS) || (part_rows_per_rank[i] % GATHER_ROWS) || part_rows_per_rank[i] <= 0 ||
            (long long)part_rows_per_rank[i] * world < part_rows[i] || (part_off[i] % 8))
            return -1;
        g.part_begin[i] = rows;
        g.rows_per_rank[i] = part_rows_per_rank[i];
        g.part_off[i] = part_off[i];
        rows += part_rows[i];
    }
    g.part_begin[n_parts] = rows;
    if (rows != N) return -1;
    g.counters = counters;
    g.target = call_index * (G2_BN / GATHER_ROWS);     // a partial last n-block still counts its real sub-units below
    for (int r = 0; r < world; ++r) g.shard[r] = reinterpret_cast<const __nv_bfloat16*>(shards[r]);
    if (N % G2_BN) return -3;                          // keep the per-block sub-unit count uniform
    // start at the n-blocks of this rank's share of the rows: with one part those are its own rows (nothing to fetch),
    // and in any case the W ranks begin their pulls at W different owners
    const int tiles_n = N / G2_BN;
    g.unit_rot = ((tiles_n * rank) / world) * (G2_BN / GATHER_ROWS);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    return a_mn ? launch_gemm_pair<true, false, true>(tmA, tmB, p, max_ctas, st, g)
                : launch_gemm_pair<false, false, true>(tmA, tmB, p, max_ctas, st, g);
}

// One part: shards[r] = rank r's rows [r*rows_per_rank, min(N,(r+1)*rows_per_rank)) of B, pitch ldb (peer pointers).
extern "C" int pb_gemm_bf16_allgather(const void* A, void* const* shards, void* b_full, void* C, const void* R, int M, int N, int K,
                                      long long lda, long long ldb, long long ldc, long long ldr, int a_mn, int out_fp32, int world,
                                      int rank, int rows_per_rank, int* counters, int call_index, int max_ctas, int* status,
                                      void* stream) {
    const int rows[1] = {N}, rpr[1] = {rows_per_rank};
    const long long off[1] = {0};
    return pb_gemm_bf16_allgather_parts(A, shards, b_full, C, R, M, N, K, lda, ldb, ldc, ldr, a_mn, out_fp32, world, rank, 1, rows, rpr, off,
                                        counters, call_index, max_ctas, status, stream);
}

// Split-K form for products with few output tiles and a long K (weight gradients): `slices` K ranges per
// tile run as separate work items and leave fp32 partial tiles in ws[slices][M][N]; pb_splitk_reduce
// then sums them (plus an optional addend) into the real output. Deterministic: no atomics.
extern "C" int pb_gemm_bf16_pair_splitk(const void* A, const void* B, float* ws, int M, int N, int K, long long lda, long long ldb,
                                        int a_mn, int b_mn, int slices, int max_ctas, int* status, void* stream) {
    using namespace pb;
    if (M <= 0 || N <= 0 || K <= 0 || slices < 1) return 0;
    if ((lda % 8) || (ldb % 8) || (N % 4) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
        (reinterpret_cast<uintptr_t>(ws) & 15))
        return -1;
    CUtensorMap tmA, tmB;
    int rc;
    if (!a_mn) rc = make_tmap_bf16_2d(&tmA, A, K, M, lda, BK, 128);
    else       rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, 64, BK);
    if (rc) return rc;
    if (!b_mn) rc = make_tmap_bf16_2d(&tmB, B, K, N, ldb, BK, 128);
    else       rc = make_tmap_bf16_2d(&tmB, B, N, K, ldb, 64, BK);
    if (rc) return rc;
    const int num_kb = (K + BK - 1) / BK;
    const int kb_per = (num_kb + slices - 1) / slices;
    GemmParams p{};
    p.M = M; p.N = N; p.K = K; p.C = ws; p.R = nullptr; p.ldc = N; p.ldr = 0; p.out_fp32 = 1; p.status = status;
    p.num_items = (num_kb + kb_per - 1) / kb_per;      // slices that really have k-blocks
    p.kb_per_split = kb_per;
    p.split_stride = (long long)M * N;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (!a_mn && !b_mn) return launch_gemm_pair<false, false>(tmA, tmB, p, max_ctas, st);
    if (!a_mn && b_mn)  return launch_gemm_pair<false, true>(tmA, tmB, p, max_ctas, st);
    if (a_mn && !b_mn)  return launch_gemm_pair<true, false>(tmA, tmB, p, max_ctas, st);
    return launch_gemm_pair<true, true>(tmA, tmB, p, max_ctas, st);
}

// number of K slices pb_gemm_bf16_pair_splitk will really use for this K and requested count
extern "C" int pb_gemm_splitk_slices(int K, int slices) {
    const int num_kb = (K + pb::BK - 1) / pb::BK;
    const int kb_per = (num_kb + slices - 1) / slices;
    return (num_kb + kb_per - 1) / kb_per;
}
