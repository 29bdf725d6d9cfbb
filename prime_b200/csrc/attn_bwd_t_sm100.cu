// Flash attention backward for head size 64: persistent, transposed-score form (sm_100a: tcgen05 + TMEM + TMA).
//
// Work item = one 128-row KV tile of one KV head; it walks every (query head of the group, query tile) pair
// that can see the tile, keeps dK/dV of the tile in TMEM, and sends dQ of each pair through a staging box and a
// bulk reduce-add (the decomposition of attn_bwd_sm100.cu). Two things differ:
//
// 1. The score tiles are computed TRANSPOSED:
//      S^T  = K Q^T,  dP^T = V dO^T            -> TMEM, lanes = kv rows, columns = query rows
//      P^T  = exp2(S^T*c - lse2[q])            -> bf16 pairs in TMEM: the A operand of dV += P^T dO as it stands
//      dS^T = P^T * (dP^T - D[q])              -> bf16 in ONE shared-memory tile, read K-major by dK += dS^T Q and
//                                                 MN-major by dQ = dS K
//    P never touches shared memory and the dV MMA reads A from tensor memory (208 KB of shared-memory traffic per
//    pair instead of 368 KB). The softmax statistics are per COLUMN here: lse2, D and the document start of the
//    pair's 128 query rows are staged in shared memory one pair ahead and read as warp-wide broadcasts.
//
// 2. The kernel is PERSISTENT: one CTA per SM takes work items from a global counter (items in kv-tile order within
//    a head, so CTAs that run at the same time share their Q/dO tiles through L2), and consecutive items are
//    pipelined into each other. Measured with one CTA per
//    item, a CTA cost 7.8 us of fixed time (launch, TMEM allocation, K/V load, pipeline fill and drain, dK/dV
//    write-out) against 1.9 us per pair, i.e. half of the kernel at 1024-token sequences. Here K/V are
//    double-buffered, so the next item's K/V load and first S^T/dP^T run under the current item's last pairs, and
//    the dK/dV write-out of an item is done by the drain warps while the next item is already being computed.
//
// 512 threads, four warpgroups (register budgets re-split with setmaxnreg):
//   warps 0-3   : warp 0 = TMA producer, warp 1 = MMA issuer (one thread)
//   warps 4-11  : softmax warps; warp w owns kv rows (TMEM lanes) 32*(w&3).. and query columns 64*((w-4)>>2)..
//   warps 12-15 : drain warps: dQ of every pair, dK/dV of every finished item
// Every wait is bounded (common.cuh); the rendezvous of the softmax warps is an mbarrier too, so a CTA that gives
// up never leaves a warp parked at a hardware barrier.
#include "attn_bwd.cuh"

namespace pb {

namespace {

struct Cfg {
    static constexpr int HD = 64;
    static constexpr int TILE_BYTES = 128 * HD * 2;      // one K / V / Q / dO tile
    static constexpr int DS_BYTES = 128 * 128 * 2;       // dS^T, two 64-column swizzle blocks
    static constexpr int STAGES = 3;
    static constexpr int DQ_STAGE_BYTES = 8 * 4096;      // two 32x32 fp32 boxes per drain warp
    static constexpr int STAT_BYTES = 2 * (128 * 4 + 128 * 4 + 128);   // [2 buffers][lse2 f32, D f32, start u8][128 query rows]
    // no alignment slack: the kernel checks that the dynamic window is 1024-byte aligned and reports an error otherwise
    static constexpr int SMEM_BYTES = TILE_BYTES * (4 + 2 * STAGES) + DS_BYTES + DQ_STAGE_BYTES + STAT_BYTES + 224;
    // tensor memory columns: all 512 are in use
    static constexpr int T_S = 0, T_DP = 128, T_DV = 256, T_DK = 320, T_DQ = 384, T_P = 448;
};
static_assert(Cfg::SMEM_BYTES <= 227 * 1024, "shared memory budget");

__device__ __forceinline__ void regs_to_64() { asm volatile("setmaxnreg.dec.sync.aligned.u32 64;"); }
__device__ __forceinline__ void regs_to_96() { asm volatile("setmaxnreg.dec.sync.aligned.u32 96;"); }
__device__ __forceinline__ void regs_to_176() { asm volatile("setmaxnreg.inc.sync.aligned.u32 176;"); }

__device__ __forceinline__ uint32_t ex2_bf16x2(uint32_t x) {
    uint32_t e;
    asm("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(e) : "r"(x));
    return e;
}

__device__ __forceinline__ void sts_u4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Position in the pair sequence of this CTA's work items. Every role keeps its own copy; the item ids come from a
// small shared-memory ring that the TMA warp fills from the global work counter.
struct Walk {
    int n;                   // ordinal of the item within this CTA
    int idx;                 // work item (>= n_items: no more work)
    int kv_tile, g, n_q;     // the item: kv tile, kv head, number of query tiles that see it
    int hq, qi;              // the pair: query head, query tile = kv_tile + qi
};

// Reads the CTA's n-th work item from the ring (bounded wait) and decodes it.
__device__ __forceinline__ void walk_load_item(Walk& w, uint32_t bar_item, const volatile int* items, volatile int* abort_flag, int* status,
                                            int n_items, int n_tiles, int G, const int* __restrict__ nq) {
    const bool good = mbar_wait(bar_item + 8 * (w.n & 3), (w.n >> 2) & 1, abort_flag, status, PB_ERR_TIMEOUT_MISC);
    w.idx = good ? items[w.n & 3] : n_items;
    if (w.idx >= n_items) return;
    w.g = w.idx / n_tiles;                 // kv tile fastest: neighbouring items share the head's Q / dO tiles
    w.kv_tile = w.idx - w.g * n_tiles;
    w.n_q = nq[w.kv_tile];
    w.hq = w.g * G;
    w.qi = 0;
}

__global__ void __launch_bounds__(512, 1)
attn_bwd_t64_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
                    const __grid_constant__ CUtensorMap tmDQ, const AttnBwdParams p) {
    constexpr int HD = Cfg::HD;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    if (base & 1023u) {
        if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, PB_ERR_TIMEOUT_MISC | 0x80);
        return;
    }
    uint8_t* gen = smem_raw;
    const uint32_t sK = base;                                    // [2]
    const uint32_t sV = sK + 2 * Cfg::TILE_BYTES;                // [2]
    const uint32_t sQ = sV + 2 * Cfg::TILE_BYTES;                // [STAGES]
    const uint32_t sDO = sQ + STAGES * Cfg::TILE_BYTES;          // [STAGES]
    const uint32_t sDS = sDO + STAGES * Cfg::TILE_BYTES;         // dS^T: [128 kv rows][128 query columns] bf16
    const uint32_t sDQ = sDS + Cfg::DS_BYTES;                    // [4 drain warps][2 boxes][32 rows][32 floats], 128B-swizzled
    float* st_lse = reinterpret_cast<float*>(gen + (sDQ - base) + Cfg::DQ_STAGE_BYTES);   // [2][128]
    float* st_D = st_lse + 256;                                                          // [2][128]
    uint8_t* st_start = reinterpret_cast<uint8_t*>(st_D + 256);                          // [2][128]: clamp(seq_start - kv0, 0, 255)
    uint64_t* bars = reinterpret_cast<uint64_t*>(st_start + 256);
    const uint32_t bar_kv = smem_u32(bars);          // [2] K and V of an item are in shared memory
    const uint32_t bar_kvempty = bar_kv + 16;        // [2] every MMA of the item that used the buffer is done
    const uint32_t bar_qfull = bar_kvempty + 16;     // [3] Q and dO of a pair are in shared memory
    const uint32_t bar_qdoempty = bar_qfull + 24;    // [3]
    const uint32_t bar_sdpfull = bar_qdoempty + 24;  // S^T and dP^T of a pair are in TMEM
    const uint32_t bar_sdpfree = bar_sdpfull + 8;    // softmax warps hold S^T and dP^T in registers (count 8)
    const uint32_t bar_pdsfull = bar_sdpfree + 8;    // P^T is in TMEM and dS^T in shared memory (count 8)
    const uint32_t bar_dqfull = bar_pdsfull + 8;     // dV/dK/dQ MMAs of a pair are done: dQ readable, P^T/dS^T reusable
    const uint32_t bar_dqempty = bar_dqfull + 8;     // drain warps have read dQ out of TMEM (count 4)
    const uint32_t bar_stat = bar_dqempty + 8;       // softmax warps: statistics buffer published / released (count 8)
    const uint32_t bar_dkvfree = bar_stat + 8;       // drain warps have read dK/dV of a finished item out of TMEM (count 4)
    const uint32_t bar_item = bar_dkvfree + 8;       // [4] ring of work-item ids: entry n & 3 holds the CTA's n-th item
    volatile int* items = reinterpret_cast<volatile int*>(bars + 21);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 23);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int G = p.H / p.KV;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_kv + 8 * s, 1);
            mbar_init(bar_kvempty + 8 * s, 1);
        }
        for (int s = 0; s < 3; ++s) {
            mbar_init(bar_qfull + 8 * s, 1);
            mbar_init(bar_qdoempty + 8 * s, 1);
        }
        mbar_init(bar_sdpfull, 1);
        mbar_init(bar_sdpfree, 8);
        mbar_init(bar_pdsfull, 8);
        mbar_init(bar_dqfull, 1);
        mbar_init(bar_dqempty, 4);
        mbar_init(bar_stat, 8);
        mbar_init(bar_dkvfree, 4);
        for (int s = 0; s < 4; ++s) mbar_init(bar_item + 8 * s, 1);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmQKV);
        tma_prefetch_desc(&tmDO);
        tma_prefetch_desc(&tmDQ);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // walker primitives (every caller is either a whole warp or a single thread; all waits are bounded)
    auto walk_load = [&](Walk& w) { walk_load_item(w, bar_item, items, abort_flag, p.status, p.n_items, p.n_tiles, G, p.nq); };
    auto walk_start = [&](Walk& w) {
        w.n = 0; w.idx = p.n_items; w.kv_tile = w.g = w.n_q = w.hq = w.qi = 0;
        walk_load(w);
    };
    auto walk_valid = [&](const Walk& w) { return w.idx < p.n_items; };
    auto walk_first = [&](const Walk& w) { return w.qi == 0 && w.hq == w.g * G; };
    auto walk_last = [&](const Walk& w) { return w.qi == w.n_q - 1 && w.hq == (w.g + 1) * G - 1; };
    auto walk_next = [&](Walk& w) -> bool {      // next pair; true when that pair belongs to another item (or there is none)
        if (++w.qi < w.n_q) return false;
        w.qi = 0;
        if (++w.hq < (w.g + 1) * G) return false;
        ++w.n;
        walk_load(w);
        return true;
    };

    if (warp < 4) {
        regs_to_64();
        if (warp == 0) {
            // ------------------------------ TMA producer ------------------------------
            // K/V of item n go to buffer n & 1 as soon as the MMAs of item n - 2 have released it, i.e. while
            // item n - 1 is still being computed; Q/dO of the pairs follow through the 3-stage ring.
            // The lane that issues the loads also feeds the item ring: item 0 is the CTA's own index, later ones come
            // from the global counter (started at gridDim.x by the pre-pass).
            auto fetch_item = [&](int n) {       // only used for item 0 (the CTA's own index)
                if (lane == 0) {
                    items[n & 3] = int(blockIdx.x);
                    mbar_arrive(bar_item + 8 * (n & 3));
                }
                __syncwarp();
            };
            auto load_kv = [&](int n, int kv_tile, int g) {
                if (lane == 0) {
                    const int kb = n & 1;
                    mbar_expect_tx(bar_kv + 8 * kb, 2 * Cfg::TILE_BYTES);
                    tma_load_2d(sK + kb * Cfg::TILE_BYTES, &tmQKV, bar_kv + 8 * kb, (p.H + g) * HD, kv_tile * 128);
                    tma_load_2d(sV + kb * Cfg::TILE_BYTES, &tmQKV, bar_kv + 8 * kb, (p.H + p.KV + g) * HD, kv_tile * 128);
                }
            };
            fetch_item(0);
            Walk w;
            walk_start(w);
            bool ok = true;
            bool kv_issued = false;          // K/V of the current item were already loaded ahead, during the previous item
            Walk ahead = w;                  // the item after the current one (only its item fields are used)
            ahead.idx = p.n_items;
            for (int j = 0; walk_valid(w) && ok; ++j) {
                const bool opens = walk_first(w);
                int next_id = 0;
                if (opens) {
                    if (!kv_issued) {
                        ok = mbar_wait(bar_kvempty + 8 * (w.n & 1), ((w.n >> 1) & 1) ^ 1, abort_flag, p.status, PB_ERR_TIMEOUT_EMPTY);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        load_kv(w.n, w.kv_tile, w.g);
                    }
                    kv_issued = false;
                    // the id of the item after this one: the atomic is issued now and its result is used only after this
                    // pair's loads are out, a whole item ahead of its use by the other roles
                    if (lane == 0) next_id = atomicAdd(p.counter, 1);
                }
                const int st = j % STAGES;
                const uint32_t ph = (j / STAGES) & 1;
                ok = mbar_wait(bar_qdoempty + 8 * st, ph ^ 1, abort_flag, p.status, PB_ERR_TIMEOUT_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (lane == 0) {
                    const int q0 = (w.kv_tile + w.qi) * 128;
                    mbar_expect_tx(bar_qfull + 8 * st, 2 * Cfg::TILE_BYTES);   // Q and dO land on one barrier
                    tma_load_2d(sQ + st * Cfg::TILE_BYTES, &tmQKV, bar_qfull + 8 * st, w.hq * HD, q0);
                    tma_load_2d(sDO + st * Cfg::TILE_BYTES, &tmDO, bar_qfull + 8 * st, w.hq * HD, q0);
                }
                __syncwarp();
                if (opens) {
                    if (lane == 0) {
                        items[(w.n + 1) & 3] = next_id;
                        mbar_arrive(bar_item + 8 * ((w.n + 1) & 3));
                    }
                    __syncwarp();
                    ahead.n = w.n + 1;
                    walk_load(ahead);
                }
                // K/V of the next item: its buffer is the one item n - 1 used; load as soon as that item's MMAs are done
                if (!kv_issued && walk_valid(ahead)) {
                    const bool free_now = mbar_try_wait(bar_kvempty + 8 * (ahead.n & 1), ((ahead.n >> 1) & 1) ^ 1);
                    if (__all_sync(0xffffffffu, free_now)) {
                        load_kv(ahead.n, ahead.kv_tile, ahead.g);
                        kv_issued = true;
                    }
                }
                walk_next(w);
            }
            if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(10000);
        } else if (warp == 1) {
            // ------------------------------ MMA issuer ------------------------------
            // One thread runs the whole loop over the flattened pair sequence of all items; barriers that are certain
            // to complete while a batch of MMAs is being issued are polled inside that batch (umma4_*_peek).
            if (lane == 0) {
                constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);    // S^T, dP^T: both operands K-major
                constexpr uint32_t idesc_dv = umma_idesc_bf16(128, HD, 0, 1);    // A = P^T in TMEM, B = dO MN-major
                constexpr uint32_t idesc_dk = umma_idesc_bf16(128, HD, 0, 1);    // A = dS^T K-major, B = Q MN-major
                constexpr uint32_t idesc_dq = umma_idesc_bf16(128, HD, 1, 1);    // A = dS (dS^T read MN-major), B = K MN-major
                const uint32_t tS = tmem_base + Cfg::T_S, tDP = tmem_base + Cfg::T_DP, tDV = tmem_base + Cfg::T_DV,
                               tDK = tmem_base + Cfg::T_DK, tDQ = tmem_base + Cfg::T_DQ, tP = tmem_base + Cfg::T_P;
                bool ok = true;
                // S^T = K Q^T and dP^T = V dO^T of pair j (Q / dO in stage j % 3, K / V in buffer kb); polls (peek, par) meanwhile
                auto issue_s_dp = [&](int j, int kb, bool q_ready, uint32_t peek, uint32_t par) -> bool {
                    const int st = j % STAGES;
                    const uint32_t ph = (j / STAGES) & 1;
                    if (!q_ready) {
                        ok = mbar_wait(bar_qfull + 8 * st, ph, abort_flag, p.status, PB_ERR_TIMEOUT_FULL);
                        if (!ok) return false;
                    }
                    tc_fence_after();
                    const uint32_t q = sQ + st * Cfg::TILE_BYTES, d = sDO + st * Cfg::TILE_BYTES;
                    umma4_f16_ss_peek(tS, umma_smem_desc(sK + kb * Cfg::TILE_BYTES, 16, 1024), umma_smem_desc(q, 16, 1024), 2, 2, idesc_s,
                                      0u, 0, 0, 0, 0, 0, 0, 0);
                    const uint32_t got = umma4_f16_ss_peek(tDP, umma_smem_desc(sV + kb * Cfg::TILE_BYTES, 16, 1024),
                                                           umma_smem_desc(d, 16, 1024), 2, 2, idesc_s, 0u, bar_sdpfull, 0, 0, peek, par, 0, 0);
                    return got & 1;
                };
                Walk cur;
                walk_start(cur);
                Walk nx = cur;
                if (walk_valid(cur)) {
                    ok = mbar_wait(bar_kv, 0, abort_flag, p.status, PB_ERR_TIMEOUT_FULL);
                    if (ok) issue_s_dp(0, 0, false, 0, 0);
                    walk_next(nx);
                }
                bool sdpfree_ready = false, qnext_ready = false;
                for (int j = 0; walk_valid(cur) && ok; ++j) {
                    const int st = j % STAGES;
                    const int kb = cur.n & 1;
                    bool pds_ready = false;
                    if (walk_valid(nx)) {
                        if (!sdpfree_ready) {
                            ok = mbar_wait(bar_sdpfree, j & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_EMPTY);
                            if (!ok) break;
                        }
                        if (walk_first(nx)) {   // the next pair opens another item: its K/V were loaded ahead
                            ok = mbar_wait(bar_kv + 8 * (nx.n & 1), (nx.n >> 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_FULL);
                            if (!ok) break;
                        }
                        pds_ready = issue_s_dp(j + 1, nx.n & 1, qnext_ready, bar_pdsfull, j & 1);
                        if (!ok) break;
                    }
                    if (!pds_ready) {
                        ok = mbar_wait(bar_pdsfull, j & 1, abort_flag, p.status, PB_ERR_TIMEOUT_MISC);
                        if (!ok) break;
                    }
                    tc_fence_after();
                    const uint32_t q = sQ + st * Cfg::TILE_BYTES, d = sDO + st * Cfg::TILE_BYTES;
                    const uint32_t kbuf = sK + kb * Cfg::TILE_BYTES;
                    const bool first = walk_first(cur), last = walk_last(cur);
                    const bool wait_dqe = j > 0;   // the drain warps have read dQ of the previous pair
                    if (first && cur.n > 0) {      // the drain warps have read dK/dV of the previous item: they may be overwritten
                        ok = mbar_wait(bar_dkvfree, (cur.n - 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_EMPTY);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    uint32_t got = 0;
                    // dV (+)= P^T dO: reduction over the 128 query rows, 16 per MMA; A comes from tensor memory
                    // (16 bf16 of every kv row = 8 columns per step). The first pair of an item overwrites.
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        got |= umma4_f16_ts_peek(tDV, tP + h * 32, umma_smem_desc(d + h * 8192, 16384, 1024), 8, 128, idesc_dv,
                                                 (!first || h) ? 1u : 0u, 0, 0, 0, (h == 0 && wait_dqe) ? bar_dqempty : 0, (j - 1) & 1, 0, 0);
                    // dK (+)= dS^T Q: A = dS^T K-major (two 64-column blocks), B = Q rows 64b.. MN-major
#pragma unroll
                    for (int b = 0; b < 2; ++b)
                        umma4_f16_ss_peek(tDK, umma_smem_desc(sDS + b * 16384, 16, 1024), umma_smem_desc(q + b * 8192, 16384, 1024),
                                          2, 128, idesc_dk, (!first || b) ? 1u : 0u, 0, 0, 0, 0, 0, 0, 0);
                    if (wait_dqe && !(got & 1)) {
                        ok = mbar_wait(bar_dqempty, (j - 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_EMPTY);
                        if (!ok) break;
                    }
                    if (wait_dqe) tc_fence_after();
                    // dQ = dS K: reduction over the 128 kv rows; the dS^T tile is read MN-major. Meanwhile poll what
                    // the next iteration needs first (a poll of a phase that never comes just reads "not yet").
                    got = umma4_f16_ss_peek(tDQ, umma_smem_desc(sDS, 16384, 1024), umma_smem_desc(kbuf, 16384, 1024), 128, 128, idesc_dq,
                                            0u, 0, 0, 0, bar_qfull + 8 * ((j + 2) % STAGES), ((j + 2) / STAGES) & 1,
                                            bar_sdpfree, (j + 1) & 1);
                    umma4_f16_ss_peek(tDQ, umma_smem_desc(sDS + 8192, 16384, 1024), umma_smem_desc(kbuf + 8192, 16384, 1024), 128, 128,
                                      idesc_dq, 1u, bar_dqfull, bar_qdoempty + 8 * st, last ? bar_kvempty + 8 * kb : 0, 0, 0, 0, 0);
                    qnext_ready = got & 1;
                    sdpfree_ready = got & 2;
                    walk_next(cur);
                    if (walk_valid(nx)) walk_next(nx);
                }
            }
            __syncwarp();
        }
    } else if (warp >= 12) {
        regs_to_96();
        // ------------------------------ dQ drain warps ------------------------------
        // dQ tile of one pair -> registers -> this warp's two staging boxes in shared memory -> bulk
        // reduce-add into the fp32 accumulator (rows past M are clipped by the tensor map)
        const int quad = warp & 3;
        const uint32_t tDQ = tmem_base + Cfg::T_DQ + (uint32_t(quad * 32) << 16);
        const uint32_t my_dq = sDQ + quad * 8192;
        uint8_t* g_dq = gen + (my_dq - base);
        const uint32_t tDKq = tmem_base + Cfg::T_DK + (uint32_t(quad * 32) << 16), tDVq = tmem_base + Cfg::T_DV + (uint32_t(quad * 32) << 16);
        bool ok = true;
        Walk w;
        walk_start(w);
        for (int j = 0; walk_valid(w) && ok; ++j) {
            ok = mbar_wait(bar_dqfull, j & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int dq_y = (w.kv_tile + w.qi) * 128 + quad * 32;
            const int dq_x = w.hq * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 32) {     // one 32-column box at a time
                uint32_t v[32];
                tmem_ld32(tDQ + c0, v);
                if (c0 == 0) {
                    if (lane == 0) tma_store_wait_read<0>();   // earlier reduce-adds have read the staging boxes
                    __syncwarp();
                }
                tmem_ld_wait();
                if (c0 == 32) {                       // dQ of this pair is out of TMEM
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_dqempty);
                }
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float4 f;
                    f.x = __uint_as_float(v[4 * q]) * p.scale;     f.y = __uint_as_float(v[4 * q + 1]) * p.scale;
                    f.z = __uint_as_float(v[4 * q + 2]) * p.scale; f.w = __uint_as_float(v[4 * q + 3]) * p.scale;
                    *reinterpret_cast<float4*>(g_dq + (c0 >> 5) * 4096 + lane * 128 + ((q ^ (lane & 7)) << 4)) = f;
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                tma_reduce_add_2d(&tmDQ, my_dq, dq_x, dq_y);
                tma_reduce_add_2d(&tmDQ, my_dq + 4096, dq_x + 32, dq_y);
                tma_store_commit();
            }
            if (walk_last(w)) {
                // the item is complete (the barrier above covers all of its MMAs): dK (scaled) and dV of its kv tile ->
                // bf16 gradient buffer, one kv row per thread, 16 columns at a time
                const int kvrow = w.kv_tile * 128 + quad * 32 + lane;
                __nv_bfloat16* dk_row = p.dqkv + (long long)kvrow * p.dqkv_stride + (p.H + w.g) * HD;
                __nv_bfloat16* dv_row = p.dqkv + (long long)kvrow * p.dqkv_stride + (p.H + p.KV + w.g) * HD;
#pragma unroll 1
                for (int c0 = 0; c0 < 64; c0 += 32) {
                    uint32_t a[32], b[32];
                    tmem_ld32(tDKq + c0, a);
                    tmem_ld32(tDVq + c0, b);
                    tmem_ld_wait();
                    if (c0 == 32) {                   // everything is in registers: the next item may overwrite dK/dV
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_dkvfree);
                    }
                    if (kvrow < p.M) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 u, x;
                            u.x = pack_bf16x2(__uint_as_float(a[i]) * p.scale, __uint_as_float(a[i + 1]) * p.scale);
                            u.y = pack_bf16x2(__uint_as_float(a[i + 2]) * p.scale, __uint_as_float(a[i + 3]) * p.scale);
                            u.z = pack_bf16x2(__uint_as_float(a[i + 4]) * p.scale, __uint_as_float(a[i + 5]) * p.scale);
                            u.w = pack_bf16x2(__uint_as_float(a[i + 6]) * p.scale, __uint_as_float(a[i + 7]) * p.scale);
                            x.x = pack_bf16x2(__uint_as_float(b[i]), __uint_as_float(b[i + 1]));
                            x.y = pack_bf16x2(__uint_as_float(b[i + 2]), __uint_as_float(b[i + 3]));
                            x.z = pack_bf16x2(__uint_as_float(b[i + 4]), __uint_as_float(b[i + 5]));
                            x.w = pack_bf16x2(__uint_as_float(b[i + 6]), __uint_as_float(b[i + 7]));
                            *reinterpret_cast<uint4*>(dk_row + c0 + i) = u;
                            *reinterpret_cast<uint4*>(dv_row + c0 + i) = x;
                        }
                    }
                }
            }
            walk_next(w);
        }
        if (lane == 0) tma_store_wait<0>();   // all reduce-adds of this warp have landed
    } else {
        regs_to_176();
        // ------------------------------ softmax / dS / epilogue warps ------------------------------
        const int quad = warp & 3;
        const int half = (warp - 4) >> 2;
        const int r = quad * 32 + lane;               // kv row of the tile == TMEM lane
        const int sid = (warp - 4) * 32 + lane;       // 0..255 among the softmax threads
        const uint32_t lane_off = uint32_t(quad * 32) << 16;
        const uint32_t tS = tmem_base + Cfg::T_S + lane_off + half * 64, tDP = tmem_base + Cfg::T_DP + lane_off + half * 64,
                       tP = tmem_base + Cfg::T_P + lane_off + half * 32;
        const float c = p.scale_log2;
        bool ok = true;
        // Statistics of a pair's query rows: threads 0..127 fetch lse2 and D of one query row each, threads
        // 128..255 its seq_start (kept as clamp(seq_start - kv0, 0, 255): a kv row r is outside the query's document
        // when r < that value). A query row past M gets lse2 = +inf, so its P is exactly 0.
        // The loaded values wait in two registers while the current pair is exponentiated; everything else about
        // the next pair is re-derived from the walker when it is published.
        auto prefetch = [&](const Walk& w, float& a, float& b) {
            const int q0 = (w.kv_tile + w.qi) * 128;
            const int row = q0 + (sid & 127);
            const bool row_ok = row < p.M;
            a = (sid < 128) ? INFINITY : __int_as_float(255);
            b = 0.f;
            if (sid < 128) {
                if (row_ok) {
                    a = p.lse2[(long long)w.hq * p.M + row];
                    b = p.D[(long long)w.hq * p.M + row];
                }
            } else if (row_ok) {
                a = __int_as_float(min(max(p.seq_start[row] - w.kv_tile * 128, 0), 255));
            }
        };
        auto publish = [&](float a, float b, int buf) {
            if (sid < 128) {
                st_lse[buf * 128 + sid] = a;
                st_D[buf * 128 + sid] = b;
            } else {
                st_start[buf * 128 + sid - 128] = uint8_t(__float_as_int(a));
            }
        };
        int n_sync = 0;
        auto stat_sync = [&]() -> bool {   // rendezvous of the eight softmax warps (bounded)
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_stat);
            bool good = mbar_wait(bar_stat, n_sync & 1, abort_flag, p.status, PB_ERR_TIMEOUT_MISC);
            ++n_sync;
            return __all_sync(0xffffffffu, good);
        };
        uint32_t sv[64], dv[64];
        auto load_sdp = [&](int j) -> bool {
            bool good = mbar_wait(bar_sdpfull, j & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
            good = __all_sync(0xffffffffu, good);
            if (!good) return false;
            tc_fence_after();
            tmem_ld32(tS, *reinterpret_cast<uint32_t(*)[32]>(sv));
            tmem_ld32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(sv + 32));
            tmem_ld32(tDP, *reinterpret_cast<uint32_t(*)[32]>(dv));
            tmem_ld32(tDP + 32, *reinterpret_cast<uint32_t(*)[32]>(dv + 32));
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sdpfree);
            return true;
        };
        // one walker, kept one pair ahead (it feeds the prefetch); the pair being computed is described by its first
        // query row, the seq_start of its last query row and its kv tile
        Walk pf;
        walk_start(pf);
        int cur_q0 = 0, cur_tls = 0, cur_tile = 0;
        bool have = walk_valid(pf);
        if (have) {
            float a, b;
            prefetch(pf, a, b);
            publish(a, b, 0);
            cur_q0 = (pf.kv_tile + pf.qi) * 128;
            cur_tls = p.seq_start[min(cur_q0 + 127, p.M - 1)];
            cur_tile = pf.kv_tile;
            ok = stat_sync();
            if (ok) ok = load_sdp(0);
            walk_next(pf);
        }
        int j = 0;
        for (; have && ok; ++j) {
            const int cur_kv0 = cur_tile * 128;
            const bool has_next = walk_valid(pf);
            float nx_a = 0.f, nx_b = 0.f;
            int nx_tls = 0;
            if (has_next) {      // global loads land while this pair is exponentiated
                prefetch(pf, nx_a, nx_b);
                nx_tls = p.seq_start[min((pf.kv_tile + pf.qi) * 128 + 127, p.M - 1)];
            }
            const int buf = j & 1;
            const float4* L = reinterpret_cast<const float4*>(st_lse + buf * 128 + half * 64);
            const float4* Dd = reinterpret_cast<const float4*>(st_D + buf * 128 + half * 64);
            const uint32_t* Ss = reinterpret_cast<const uint32_t*>(st_start + buf * 128 + half * 64);
            // Exponentials are taken two at a time on packed bf16 pairs (ex2.approx.bf16x2): the result is
            // P^T as the MMA will read it, and dS^T is formed from those same rounded values.
            const bool need_mask = (cur_kv0 + 127 > cur_q0) || (cur_kv0 < cur_tls);
            if (need_mask) {
                const int dq = cur_q0 + half * 64 - cur_kv0;     // query column i is query row kv0 + dq + i: visible when r <= dq + i
#pragma unroll
                for (int i = 0; i < 64; i += 4) {
                    const float4 l4 = L[i >> 2];
                    const float4 d4 = Dd[i >> 2];
                    const uint32_t s4 = Ss[i >> 2];
                    float x0 = __uint_as_float(sv[i]) * c - l4.x, x1 = __uint_as_float(sv[i + 1]) * c - l4.y;
                    float x2 = __uint_as_float(sv[i + 2]) * c - l4.z, x3 = __uint_as_float(sv[i + 3]) * c - l4.w;
                    if (r > dq + i || r < int(s4 & 0xff)) x0 = -INFINITY;
                    if (r > dq + i + 1 || r < int((s4 >> 8) & 0xff)) x1 = -INFINITY;
                    if (r > dq + i + 2 || r < int((s4 >> 16) & 0xff)) x2 = -INFINITY;
                    if (r > dq + i + 3 || r < int(s4 >> 24)) x3 = -INFINITY;
                    const uint32_t e0 = ex2_bf16x2(pack_bf16x2(x0, x1)), e1 = ex2_bf16x2(pack_bf16x2(x2, x3));
                    const float g0 = __uint_as_float(e0 << 16) * (__uint_as_float(dv[i]) - d4.x);
                    const float g1 = __uint_as_float(e0 & 0xffff0000u) * (__uint_as_float(dv[i + 1]) - d4.y);
                    const float g2 = __uint_as_float(e1 << 16) * (__uint_as_float(dv[i + 2]) - d4.z);
                    const float g3 = __uint_as_float(e1 & 0xffff0000u) * (__uint_as_float(dv[i + 3]) - d4.w);
                    sv[i >> 1] = e0; sv[(i >> 1) + 1] = e1;
                    dv[i >> 1] = pack_bf16x2(g0, g1); dv[(i >> 1) + 1] = pack_bf16x2(g2, g3);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 64; i += 4) {
                    const float4 l4 = L[i >> 2];
                    const float4 d4 = Dd[i >> 2];
                    const float x0 = __uint_as_float(sv[i]) * c - l4.x, x1 = __uint_as_float(sv[i + 1]) * c - l4.y;
                    const float x2 = __uint_as_float(sv[i + 2]) * c - l4.z, x3 = __uint_as_float(sv[i + 3]) * c - l4.w;
                    const uint32_t e0 = ex2_bf16x2(pack_bf16x2(x0, x1)), e1 = ex2_bf16x2(pack_bf16x2(x2, x3));
                    const float g0 = __uint_as_float(e0 << 16) * (__uint_as_float(dv[i]) - d4.x);
                    const float g1 = __uint_as_float(e0 & 0xffff0000u) * (__uint_as_float(dv[i + 1]) - d4.y);
                    const float g2 = __uint_as_float(e1 << 16) * (__uint_as_float(dv[i + 2]) - d4.z);
                    const float g3 = __uint_as_float(e1 & 0xffff0000u) * (__uint_as_float(dv[i + 3]) - d4.w);
                    sv[i >> 1] = e0; sv[(i >> 1) + 1] = e1;
                    dv[i >> 1] = pack_bf16x2(g0, g1); dv[(i >> 1) + 1] = pack_bf16x2(g2, g3);
                }
            }
            if (j > 0) {
                // the MMAs of the previous pair have read its P^T out of tensor memory and its dS^T out of shared memory
                ok = mbar_wait(bar_dqfull, (j - 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
            }
            // P^T: 64 query columns of this kv row = 32 packed words -> tensor memory
            tmem_st32(tP, *reinterpret_cast<uint32_t(*)[32]>(sv));
            // dS^T: the same 64 columns = one 128-byte row of swizzle block `half`
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const uint32_t off = half * 16384 + r * 128 + ((q ^ (r & 7)) << 4);
                sts_u4(sDS + off, dv[4 * q], dv[4 * q + 1], dv[4 * q + 2], dv[4 * q + 3]);
            }
            tmem_st_wait();
            tc_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_pdsfull);
            have = has_next;
            if (has_next) {
                publish(nx_a, nx_b, buf ^ 1);
                cur_q0 = (pf.kv_tile + pf.qi) * 128; cur_tls = nx_tls; cur_tile = pf.kv_tile;
                ok = stat_sync();      // everyone is done reading `buf`; `buf ^ 1` is complete
                if (!ok) break;
                ok = load_sdp(j + 1);
                walk_next(pf);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// nq[kv_tile] = number of query tiles that can see the kv tile: the diagonal tile plus every later tile whose first
// row's sequence starts at or before the tile's last kv row (seq_start is non-decreasing). One warp per kv tile, 32
// candidate tiles per step.
__global__ void attn_bwd_span_kernel(const int* __restrict__ seq_start, int n_tiles, int* __restrict__ nq, int* counter, int first_free) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *counter = first_free;   // items below first_free are taken by CTA index
    const int kv_tile = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (kv_tile >= n_tiles) return;
    const int kv_last = kv_tile * 128 + 127;
    int n_q = 1;
    for (int t0 = kv_tile + 1; t0 < n_tiles; t0 += 32) {
        const int t = t0 + lane;
        const bool sees = t < n_tiles && seq_start[t * 128] <= kv_last;
        const uint32_t m = __ballot_sync(0xffffffffu, sees);
        const int run = __ffs(~m) - 1;
        if (run >= 0) { n_q += run; break; }
        n_q += 32;
    }
    if (lane == 0) nq[kv_tile] = n_q;
}

}  // namespace

int launch_attn_bwd_t64(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tdq, const AttnBwdParams& p,
                        int* nq_scratch, cudaStream_t st) {
    static int n_sm = 0;
    if (n_sm == 0) {
        if (cudaFuncSetAttribute(attn_bwd_t64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
            return -20;
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return -21;
    }
    AttnBwdParams q = p;
    q.nq = nq_scratch;
    q.counter = nq_scratch + p.n_tiles;
    q.n_items = p.n_tiles * p.KV;
    const int grid = q.n_items < n_sm ? q.n_items : n_sm;
    attn_bwd_span_kernel<<<(p.n_tiles * 32 + 255) / 256, 256, 0, st>>>(p.seq_start, p.n_tiles, nq_scratch, q.counter, grid);
    attn_bwd_t64_kernel<<<grid, 512, Cfg::SMEM_BYTES, st>>>(tq, tdo, tdq, q);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

}  // namespace pb
