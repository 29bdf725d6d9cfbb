// Flash attention backward (causal / document mask, GQA) for sm_100a on tcgen05 + TMEM + TMA.
//
// A work item is one 128-row KV tile of one KV head; the CTA that holds it walks every (query head of the
// group, query tile) pair that can see it. Per pair (all MMAs are 128-row tcgen05 instructions):
//   S  = Q K^T,  dP = dO V^T                 -> TMEM
//   P  = exp2(S*c - lse2),  dS = P * (dP - D) -> bf16 in shared memory (softmax warps)
//   dV += P^T dO,  dK += dS^T Q               -> TMEM accumulators kept for the whole item
//   dQ  = dS K                                -> TMEM -> shared memory -> bulk reduce-add (TMA) into dq_acc
// For head size 64 the pairs are software-pipelined: the tensor core computes S/dP of pair i+1 and dV/dK/dQ of
// pair i-1 while the softmax warps work on pair i from registers.
// D[h, m] = rowsum(dO * O) comes from a small pre-pass. dK/dV of a KV head are reduced over the
// query heads of its group inside the CTA (no repeat_kv materialisation, no cross-CTA atomics
// for them). The same shared-memory tile is consumed K-major by one MMA and MN-major by another
// (e.g. Q is A of S and B of dK), which the 128-byte-swizzled layout allows without a copy.
// Gradient semantics match autograd through the reference attention
// (models/llama/model.py:282-302) for scores scaled by `scale`.
#include "common.cuh"

namespace pb {

struct AttnBwdParams {
    int M, H, KV, n_tiles;
    const int* seq_start;
    const float* lse2;     // [H, M]
    const float* D;        // [H, M]
    float* dq_acc;         // [M, H*HD] fp32, zero-initialised by the caller
    __nv_bfloat16* dqkv;   // [M, (H+2KV)*HD]; the backward kernel writes the k and v column blocks
    long long dqkv_stride;
    float scale, scale_log2;
    int* status;
    // query-tile count per kv tile (set by a pre-pass of the launch) and work-item count (= n_tiles * KV)
    int* nq;
    int n_items;
    int* counter;          // the global work counter (next item number)
};

template <int HD>
struct AttnBwdCfg {
    static constexpr int TILE_BYTES = 128 * HD * 2;
    static constexpr int PS_BYTES = 128 * 128 * 2;
    static constexpr int STAGES = (HD == 64) ? 3 : 1;
    // HD=64: S/dP of pair it+1 are issued as soon as the softmax warps hold pair it in registers
    static constexpr bool PIPE = (HD == 64);
    static constexpr int DQ_STAGE_BYTES = 8 * 4096;   // one 32-row x 32-float box per softmax warp
    static constexpr int SMEM_BYTES = TILE_BYTES * (2 + 2 * STAGES) + 2 * PS_BYTES + DQ_STAGE_BYTES + 1024 + 256;
    static constexpr int T_S = 0, T_DP = 128;
    static constexpr int T_DV = 256, T_DK = 256 + HD;
    static constexpr int T_DQ = (HD == 64) ? 384 : 0;   // HD=128: dQ reuses the S columns
    static constexpr bool DQ_ALIASES_S = (HD != 64);
};

__device__ __forceinline__ void reg_dealloc_64() { asm volatile("setmaxnreg.dec.sync.aligned.u32 64;"); }
__device__ __forceinline__ void reg_dealloc_88() { asm volatile("setmaxnreg.dec.sync.aligned.u32 88;"); }
__device__ __forceinline__ void reg_alloc_176() { asm volatile("setmaxnreg.inc.sync.aligned.u32 176;"); }

// A work item is one (kv tile, kv head). The grid is one CTA per SM; every CTA draws items from a global counter
// (the producer warp does, and hands the numbers to the other warps through a four-entry ring in shared memory), so
// barriers, tensor memory and the Q/dO ring are set up once per SM and the next item's K/V/Q/dO loads run under the
// current item's dK/dV write-out. Items are numbered head by head, kv tiles in row order, so the CTAs that run at the
// same time share Q, dO and the dQ accumulator rows in L2.
struct BwdItem {
    int kv_tile, g;
};

__device__ __forceinline__ BwdItem bwd_item_of(const AttnBwdParams& p, int idx) {
    BwdItem it;
    it.g = idx / p.n_tiles;
    it.kv_tile = idx - it.g * p.n_tiles;
    return it;
}

// 512 threads in four warpgroups (register budgets are re-split with setmaxnreg):
//   warps 0-3   : warp 0 = TMA producer, warp 1 = MMA issuer (2 and 3 only hold the warpgroup together)
//   warps 4-11  : softmax warps; warp w reads TMEM lane quadrant w & 3 and column half (w - 4) >> 2
//   warps 12-15 : dQ drain warps; warp w moves the 32 query rows of quadrant w & 3 to dq_acc
template <int HD>
__global__ void __launch_bounds__(512, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
                const __grid_constant__ CUtensorMap tmDQ, const AttnBwdParams p) {
    using Cfg = AttnBwdCfg<HD>;
    constexpr int NB = HD / 64;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sK = base;
    const uint32_t sV = sK + Cfg::TILE_BYTES;
    const uint32_t sQ = sV + Cfg::TILE_BYTES;                    // [STAGES]
    const uint32_t sDO = sQ + STAGES * Cfg::TILE_BYTES;          // [STAGES]
    const uint32_t sP = sDO + STAGES * Cfg::TILE_BYTES;
    const uint32_t sDS = sP + Cfg::PS_BYTES;
    uint8_t* gP = gen + (sP - base);
    uint8_t* gDS = gen + (sDS - base);
    const uint32_t sDQ = sDS + Cfg::PS_BYTES;                    // [4 drain warps][2 boxes][32 rows][32 floats], 128B-swizzled
    uint64_t* bars = reinterpret_cast<uint64_t*>(gen + (sDQ - base) + Cfg::DQ_STAGE_BYTES);
    const uint32_t bar_kv = smem_u32(bars);
    const uint32_t bar_qfull = bar_kv + 8;           // [3] Q and dO of a pair are in shared memory
    const uint32_t bar_qdoempty = bar_qfull + 24;    // [3]
    const uint32_t bar_sdpfull = bar_qdoempty + 24;  // S and dP of a pair are in TMEM
    const uint32_t bar_sdpfree = bar_sdpfull + 8;    // softmax warps hold S and dP in registers (count 8)
    const uint32_t bar_pdsfull = bar_sdpfree + 8;    // P and dS of a pair are in shared memory (count 8)
    const uint32_t bar_dqfull = bar_pdsfull + 8;     // dV/dK/dQ MMAs of a pair are done: dQ readable, P/dS reusable
    const uint32_t bar_dqempty = bar_dqfull + 8;     // drain warps have read dQ out of TMEM (count 4)
    const uint32_t bar_final = bar_dqempty + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    ItemRing items;
    items.bar_full = bar_final + 8;                 // [4]
    items.bar_empty = items.bar_full + 32;          // [4]
    items.ring = reinterpret_cast<volatile int*>(tmem_slot + 2);
    items.abort_flag = abort_flag;
    items.status = p.status;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.H / p.KV;

    if (threadIdx.x == 0) {
        mbar_init(bar_kv, 1);
        for (int s = 0; s < 3; ++s) {
            mbar_init(bar_qfull + 8 * s, 1);
            mbar_init(bar_qdoempty + 8 * s, 1);
        }
        mbar_init(bar_sdpfull, 1);
        mbar_init(bar_sdpfree, 8);
        mbar_init(bar_pdsfull, 8);
        mbar_init(bar_dqfull, 1);
        mbar_init(bar_dqempty, 4);
        mbar_init(bar_final, 1);
        for (int s = 0; s < 4; ++s) {
            mbar_init(items.bar_full + 8 * s, 1);
            mbar_init(items.bar_empty + 8 * s, 13);   // MMA thread, eight softmax warps, four drain warps
        }
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

    if (warp < 4) {
        reg_dealloc_64();
        if (warp == 0) {
            // ------------------------------ TMA producer ------------------------------
            bool ok = true;
            uint32_t gi = 0;          // running pair count: ring stage and barrier parities carry over from item to item
            int idx = items.publish(0, p.counter, p.n_items);
            for (int k = 0; ok && idx >= 0; ++k) {
                const BwdItem item = bwd_item_of(p, idx);
                const int kv0 = item.kv_tile * 128;
                const int n_q = p.nq[item.kv_tile];
                if (k > 0) {   // every MMA of the previous item has retired: K and V may be replaced
                    ok = mbar_wait(bar_final, (k - 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                if (lane == 0) {
                    mbar_expect_tx(bar_kv, 2 * Cfg::TILE_BYTES);
#pragma unroll
                    for (int b = 0; b < NB; ++b) {
                        tma_load_2d(sK + b * 16384, &tmQKV, bar_kv, (p.H + item.g) * HD + 64 * b, kv0);
                        tma_load_2d(sV + b * 16384, &tmQKV, bar_kv, (p.H + p.KV + item.g) * HD + 64 * b, kv0);
                    }
                }
                int hq = item.g * G, qi = 0;
                const int n_it = n_q * G;
                for (int it = 0; it < n_it && ok; ++it, ++gi) {
                    const int st = gi % STAGES;
                    const uint32_t ph = (gi / STAGES) & 1;
                    ok = mbar_wait(bar_qdoempty + 8 * st, ph ^ 1, abort_flag, p.status, PB_ERR_TIMEOUT_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    if (lane == 0) {
                        const int q0 = (item.kv_tile + qi) * 128;
                        mbar_expect_tx(bar_qfull + 8 * st, 2 * Cfg::TILE_BYTES);   // Q and dO land on one barrier
#pragma unroll
                        for (int b = 0; b < NB; ++b)
                            tma_load_2d(sQ + st * Cfg::TILE_BYTES + b * 16384, &tmQKV, bar_qfull + 8 * st, hq * HD + 64 * b, q0);
#pragma unroll
                        for (int b = 0; b < NB; ++b)
                            tma_load_2d(sDO + st * Cfg::TILE_BYTES + b * 16384, &tmDO, bar_qfull + 8 * st, hq * HD + 64 * b, q0);
                    }
                    __syncwarp();
                    if (++qi == n_q) { qi = 0; ++hq; }
                }
                if (!ok) break;
                // The next item is drawn only now, when this item's last loads are in flight: a CTA that is still busy
                // with a heavy item leaves the counter to the others. The other warps ask for it after their last pair.
                idx = items.publish(k + 1, p.counter, p.n_items);
                if (idx == -2) ok = false;
            }
            if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(10000);
        } else if (warp == 1) {
            // ------------------------------ MMA issuer ------------------------------
            // One thread runs the whole loop. Barriers that are certain to complete while a batch of
            // MMAs is being issued are polled inside that batch (umma4_f16_ss_peek), so their latency
            // is not paid between batches.
            if (lane == 0) {
                constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
                constexpr uint32_t idesc_kv = umma_idesc_bf16(128, HD, 1, 1);   // dV, dK: both operands MN-major
                constexpr uint32_t idesc_dq = umma_idesc_bf16(128, HD, 0, 1);
                const uint32_t tS = tmem_base + Cfg::T_S, tDP = tmem_base + Cfg::T_DP, tDV = tmem_base + Cfg::T_DV,
                               tDK = tmem_base + Cfg::T_DK, tDQ = tmem_base + Cfg::T_DQ;
                bool ok = true;
                // S = Q K^T and dP = dO V^T of running pair gi (operands in stage gi % STAGES); polls (peek, par) meanwhile
                auto issue_s_dp = [&](uint32_t gi, bool q_ready, uint32_t peek, uint32_t par) -> bool {
                    const int st = gi % STAGES;
                    const uint32_t ph = (gi / STAGES) & 1;
                    if (!q_ready) {
                        ok = mbar_wait(bar_qfull + 8 * st, ph, abort_flag, p.status, PB_ERR_TIMEOUT_FULL);
                        if (!ok) return false;
                    }
                    if (Cfg::DQ_ALIASES_S && gi > 0) {
                        ok = mbar_wait(bar_dqempty, (gi - 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_EMPTY);
                        if (!ok) return false;
                    }
                    tc_fence_after();
                    const uint32_t q = sQ + st * Cfg::TILE_BYTES, d = sDO + st * Cfg::TILE_BYTES;
                    uint32_t got = 0;
#pragma unroll
                    for (int b = 0; b < NB; ++b)
                        umma4_f16_ss_peek(tS, umma_smem_desc(q + b * 16384, 16, 1024), umma_smem_desc(sK + b * 16384, 16, 1024), 2, 2,
                                          idesc_s, b ? 1u : 0u, 0, 0, 0, 0, 0, 0, 0);
#pragma unroll
                    for (int b = 0; b < NB; ++b)
                        got |= umma4_f16_ss_peek(tDP, umma_smem_desc(d + b * 16384, 16, 1024), umma_smem_desc(sV + b * 16384, 16, 1024), 2, 2,
                                                 idesc_s, b ? 1u : 0u, b == NB - 1 ? bar_sdpfull : 0, 0, 0,
                                                 b == NB - 1 ? peek : 0, par, 0, 0);
                    return got & 1;
                };
                uint32_t gi = 0;      // running pair count over all items of this CTA
                for (int k = 0; ok; ++k) {
                    const int idx = items.take_thread(k);
                    if (idx < 0) break;
                    const int n_it = p.nq[bwd_item_of(p, idx).kv_tile] * G;
                    ok = mbar_wait(bar_kv, k & 1, abort_flag, p.status, PB_ERR_TIMEOUT_FULL);
                    if (!ok) break;
                    if (Cfg::PIPE && gi > 0) {   // the softmax warps hold the previous item's last pair in registers (long since)
                        ok = mbar_wait(bar_sdpfree, (gi - 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_EMPTY);
                        if (!ok) break;
                    }
                    issue_s_dp(gi, false, 0, 0);
                    bool sdpfree_ready = false, qnext_ready = false;
                    for (int it = 0; it < n_it && ok; ++it, ++gi) {
                        const int st = gi % STAGES;
                        bool pds_ready = false;
                        if (Cfg::PIPE && it + 1 < n_it) {
                            if (!sdpfree_ready) {
                                ok = mbar_wait(bar_sdpfree, gi & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_EMPTY);
                                if (!ok) break;
                            }
                            pds_ready = issue_s_dp(gi + 1, qnext_ready, bar_pdsfull, gi & 1);
                            if (!ok) break;
                        }
                        if (!pds_ready) {
                            ok = mbar_wait(bar_pdsfull, gi & 1, abort_flag, p.status, PB_ERR_TIMEOUT_MISC);
                            if (!ok) break;
                        }
                        tc_fence_after();
                        const uint32_t q = sQ + st * Cfg::TILE_BYTES, d = sDO + st * Cfg::TILE_BYTES;
                        const bool wait_dqe = !Cfg::DQ_ALIASES_S && gi > 0;   // the drain warps have read dQ of the previous pair
                        uint32_t got = 0;
                        // dV += P^T dO, dK += dS^T Q: reduction over the 128 query rows, 16 per MMA; the first pair of an
                        // item starts new accumulators (the softmax warps wrote the previous item's dK/dV out before they
                        // signalled this pair's P and dS)
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            got |= umma4_f16_ss_peek(tDV, umma_smem_desc(sP + h * 8192, 16384, 1024), umma_smem_desc(d + h * 8192, 16384, 1024),
                                                     128, 128, idesc_kv, (it | h) ? 1u : 0u, 0, 0, 0,
                                                     (h == 0 && wait_dqe) ? bar_dqempty : 0, (gi - 1) & 1, 0, 0);
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            umma4_f16_ss_peek(tDK, umma_smem_desc(sDS + h * 8192, 16384, 1024), umma_smem_desc(q + h * 8192, 16384, 1024),
                                              128, 128, idesc_kv, (it | h) ? 1u : 0u, 0, 0, 0, 0, 0, 0, 0);
                        if (wait_dqe && !(got & 1)) {
                            ok = mbar_wait(bar_dqempty, (gi - 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_EMPTY);
                            if (!ok) break;
                        }
                        if (wait_dqe) tc_fence_after();
                        // dQ = dS K: reduction over the 128 kv rows. Meanwhile poll what the next iteration needs first.
                        const int nx = Cfg::PIPE ? it + 2 : it + 1;            // pair (of this item) whose Q/dO stage is needed next
                        const uint32_t gnx = gi + (Cfg::PIPE ? 2 : 1);
                        const bool peek_q = nx < n_it;
                        const bool peek_free = Cfg::PIPE && it + 2 < n_it;
                        got = umma4_f16_ss_peek(tDQ, umma_smem_desc(sDS, 16, 1024), umma_smem_desc(sK, 16384, 1024), 2, 128, idesc_dq, 0u,
                                                0, 0, 0, peek_q ? bar_qfull + 8 * (gnx % STAGES) : 0, (gnx / STAGES) & 1,
                                                peek_free ? bar_sdpfree : 0, (gi + 1) & 1);
                        umma4_f16_ss_peek(tDQ, umma_smem_desc(sDS + 16384, 16, 1024), umma_smem_desc(sK + 8192, 16384, 1024), 2, 128, idesc_dq,
                                          1u, bar_dqfull, bar_qdoempty + 8 * st, it == n_it - 1 ? bar_final : 0, 0, 0, 0, 0);
                        qnext_ready = got & 1;
                        sdpfree_ready = got & 2;
                        if (!Cfg::PIPE && it + 1 < n_it) issue_s_dp(gi + 1, qnext_ready, 0, 0);
                    }
                }
            }
            __syncwarp();
        }
    } else if (warp >= 12) {
        reg_dealloc_88();
        // ------------------------------ dQ drain warps ------------------------------
        // dQ tile of one pair -> registers -> this warp's two staging boxes in shared memory -> bulk
        // reduce-add into the fp32 accumulator (rows past M are clipped by the tensor map)
        const int quad = warp & 3;
        const uint32_t tDQ = tmem_base + Cfg::T_DQ + (uint32_t(quad * 32) << 16);
        const uint32_t my_dq = sDQ + quad * 8192;
        uint8_t* g_dq = gen + (my_dq - base);
        bool ok = true;
        uint32_t gi = 0;
        for (int k = 0; ok; ++k) {
            const int idx = items.take(k);
            if (idx < 0) break;
            const BwdItem item = bwd_item_of(p, idx);
            const int n_q = p.nq[item.kv_tile];
            const int n_it = n_q * G;
            int hq = item.g * G, qi = 0;
            for (int it = 0; it < n_it && ok; ++it, ++gi) {
                ok = mbar_wait(bar_dqfull, gi & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const int dq_y = (item.kv_tile + qi) * 128 + quad * 32;
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 64) {
                    uint32_t v[64];
                    tmem_ld32(tDQ + c0, *reinterpret_cast<uint32_t(*)[32]>(v));
                    tmem_ld32(tDQ + c0 + 32, *reinterpret_cast<uint32_t(*)[32]>(v + 32));
                    if (lane == 0) tma_store_wait_read<0>();   // earlier reduce-adds have read the staging boxes
                    __syncwarp();
                    tmem_ld_wait();
                    if (c0 + 64 >= HD) {   // dQ of this pair is out of TMEM
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_dqempty);
                    }
#pragma unroll
                    for (int q = 0; q < 16; ++q) {
                        float4 f;
                        f.x = __uint_as_float(v[4 * q]) * p.scale;     f.y = __uint_as_float(v[4 * q + 1]) * p.scale;
                        f.z = __uint_as_float(v[4 * q + 2]) * p.scale; f.w = __uint_as_float(v[4 * q + 3]) * p.scale;
                        *reinterpret_cast<float4*>(g_dq + (q >> 3) * 4096 + lane * 128 + (((q & 7) ^ (lane & 7)) << 4)) = f;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_reduce_add_2d(&tmDQ, my_dq, hq * HD + c0, dq_y);
                        tma_reduce_add_2d(&tmDQ, my_dq + 4096, hq * HD + c0 + 32, dq_y);
                        tma_store_commit();
                    }
                }
                if (++qi == n_q) { qi = 0; ++hq; }
            }
        }
        if (lane == 0) tma_store_wait<0>();   // all reduce-adds of this warp have landed
    } else {
        reg_alloc_176();
        // ------------------------------ softmax / dS / epilogue warps ------------------------------
        // Eight warps: warp w reads TMEM lane quadrant w & 3 (a hardware rule) and takes column half
        // (w - 4) >> 2 of every 128-wide row, so two warps share each query row of the tile.
        const int quad = warp & 3;
        const int half = (warp - 4) >> 2;
        const int r = quad * 32 + lane;
        const uint32_t lane_off = uint32_t(quad * 32) << 16;
        const uint32_t tS = tmem_base + Cfg::T_S + lane_off, tDP = tmem_base + Cfg::T_DP + lane_off,
                       tDV = tmem_base + Cfg::T_DV + lane_off, tDK = tmem_base + Cfg::T_DK + lane_off;
        const float c = p.scale_log2;
        bool ok = true;
        // Per (head, query tile) pair: this thread's row constants, then its 64 S and 64 dP values in
        // registers. With Cfg::PIPE the pair after the one being exponentiated is already in TMEM.
        struct RowCtx {
            float lse, Dr;
            int my_start;
            int q0, tile_last_start;
        };
        // (query head, query tile) of the pair whose row constants are loaded next, inside the current item
        int kv_tile = 0, n_q = 0, hq_n = 0, qi_n = 0;
        auto row_ctx = [&]() {
            RowCtx x;
            const int q0 = (kv_tile + qi_n) * 128;
            const int row = q0 + r;
            const bool row_ok = row < p.M;
            x.lse = row_ok ? p.lse2[(long long)hq_n * p.M + row] : 0.f;
            x.Dr = row_ok ? p.D[(long long)hq_n * p.M + row] : 0.f;
            x.my_start = row_ok ? p.seq_start[row] : 0x7fffffff;   // a row past M sees no kv position
            x.q0 = q0;
            x.tile_last_start = p.seq_start[min(q0 + 127, p.M - 1)];
            if (++qi_n == n_q) { qi_n = 0; ++hq_n; }
            return x;
        };
        uint32_t sv[64], dv[64];
        auto load_sdp = [&](uint32_t gi) -> bool {
            bool good = mbar_wait(bar_sdpfull, gi & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
            good = __all_sync(0xffffffffu, good);
            if (!good) return false;
            tc_fence_after();
            tmem_ld32(tS + half * 64, *reinterpret_cast<uint32_t(*)[32]>(sv));
            tmem_ld32(tS + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(sv + 32));
            tmem_ld32(tDP + half * 64, *reinterpret_cast<uint32_t(*)[32]>(dv));
            tmem_ld32(tDP + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(dv + 32));
            tmem_ld_wait();
            if (Cfg::PIPE) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_sdpfree);
            }
            return true;
        };
        RowCtx cur = {}, nxt = {};
        uint32_t gi = 0;
        BwdItem item = {};
        int idx = items.take(0);
        bool have = idx >= 0;
        if (have) {
            item = bwd_item_of(p, idx);
            kv_tile = item.kv_tile; n_q = p.nq[kv_tile]; hq_n = item.g * G; qi_n = 0;
            cur = row_ctx();
        }
        for (int k = 0; have && ok; ++k) {
            const int kv0 = kv_tile * 128;
            const int g = item.g;
            int left = n_q * G;                 // pairs of this item not yet started
            ok = load_sdp(gi);
            while (ok) {
                --left;
                if (left) nxt = row_ctx();      // global loads land while this pair is exponentiated
                const int row = cur.q0 + r;
                // Exponentials are taken two at a time on packed bf16 pairs (ex2.approx.bf16x2): the result is
                // P as the MMA will read it, and dS is formed from those same rounded values.
                const bool need_mask = (kv0 + 127 > cur.q0) || (kv0 < cur.tile_last_start) || (cur.q0 + 127 >= p.M);
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 64; i += 2) {
                        const int s0 = kv0 + half * 64 + i;
                        float x0 = __uint_as_float(sv[i]) * c - cur.lse;
                        float x1 = __uint_as_float(sv[i + 1]) * c - cur.lse;
                        if (s0 > row || s0 < cur.my_start) x0 = -INFINITY;
                        if (s0 + 1 > row || s0 + 1 < cur.my_start) x1 = -INFINITY;
                        uint32_t e;
                        asm("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(e) : "r"(pack_bf16x2(x0, x1)));
                        const float d0 = __uint_as_float(e << 16) * (__uint_as_float(dv[i]) - cur.Dr);
                        const float d1 = __uint_as_float(e & 0xffff0000u) * (__uint_as_float(dv[i + 1]) - cur.Dr);
                        sv[i >> 1] = e;
                        dv[i >> 1] = pack_bf16x2(d0, d1);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 64; i += 2) {
                        const float x0 = __uint_as_float(sv[i]) * c - cur.lse;
                        const float x1 = __uint_as_float(sv[i + 1]) * c - cur.lse;
                        uint32_t e;
                        asm("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(e) : "r"(pack_bf16x2(x0, x1)));
                        const float d0 = __uint_as_float(e << 16) * (__uint_as_float(dv[i]) - cur.Dr);
                        const float d1 = __uint_as_float(e & 0xffff0000u) * (__uint_as_float(dv[i + 1]) - cur.Dr);
                        sv[i >> 1] = e;
                        dv[i >> 1] = pack_bf16x2(d0, d1);
                    }
                }
                if (gi > 0) {
                    // the MMAs of the previous pair have read its P/dS out of shared memory
                    ok = mbar_wait(bar_dqfull, (gi - 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int chunk = half * 8 + q;
                    const uint32_t off = (chunk >> 3) * 16384 + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
                    *reinterpret_cast<uint4*>(gP + off) = make_uint4(sv[4 * q], sv[4 * q + 1], sv[4 * q + 2], sv[4 * q + 3]);
                    *reinterpret_cast<uint4*>(gDS + off) = make_uint4(dv[4 * q], dv[4 * q + 1], dv[4 * q + 2], dv[4 * q + 3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_pdsfull);
                ++gi;
                if (!left) break;
                cur = nxt;
                ok = load_sdp(gi);
            }
            if (!ok) break;
            // dK (scaled) and dV of this kv tile -> bf16 gradient buffer, once every MMA of the item has retired
            ok = mbar_wait(bar_final, k & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            // the next item's first row constants are requested before the write-out, so they arrive under it
            idx = items.take(k + 1);
            have = idx >= 0;
            if (have) {
                item = bwd_item_of(p, idx);
                kv_tile = item.kv_tile; n_q = p.nq[kv_tile]; hq_n = item.g * G; qi_n = 0;
                cur = row_ctx();
            }
            tc_fence_after();
            const int row = kv0 + r;
            __nv_bfloat16* dk_row = p.dqkv + (long long)row * p.dqkv_stride + (p.H + g) * HD;
            __nv_bfloat16* dv_row = p.dqkv + (long long)row * p.dqkv_stride + (p.H + p.KV + g) * HD;
#pragma unroll 1
            for (int cidx = half * (HD / 2); cidx < (half + 1) * (HD / 2); cidx += 32) {
                uint32_t a[32], b[32];
                tmem_ld32(tDK + cidx, a);
                tmem_ld32(tDV + cidx, b);
                tmem_ld_wait();
                if (row < p.M) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 u, w;
                        u.x = pack_bf16x2(__uint_as_float(a[i]) * p.scale, __uint_as_float(a[i + 1]) * p.scale);
                        u.y = pack_bf16x2(__uint_as_float(a[i + 2]) * p.scale, __uint_as_float(a[i + 3]) * p.scale);
                        u.z = pack_bf16x2(__uint_as_float(a[i + 4]) * p.scale, __uint_as_float(a[i + 5]) * p.scale);
                        u.w = pack_bf16x2(__uint_as_float(a[i + 6]) * p.scale, __uint_as_float(a[i + 7]) * p.scale);
                        w.x = pack_bf16x2(__uint_as_float(b[i]), __uint_as_float(b[i + 1]));
                        w.y = pack_bf16x2(__uint_as_float(b[i + 2]), __uint_as_float(b[i + 3]));
                        w.z = pack_bf16x2(__uint_as_float(b[i + 4]), __uint_as_float(b[i + 5]));
                        w.w = pack_bf16x2(__uint_as_float(b[i + 6]), __uint_as_float(b[i + 7]));
                        *reinterpret_cast<uint4*>(dk_row + cidx + i) = u;
                        *reinterpret_cast<uint4*>(dv_row + cidx + i) = w;
                    }
                }
            }
            tc_fence_before();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// D[h, m] = sum_d dO[m, h*HD + d] * O[m, h*HD + d]. HD/8 consecutive lanes share one (m, h) row and
// load 16 bytes each; every thread keeps four rows in flight.
template <int HD>
__global__ void __launch_bounds__(256) attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                                            float* __restrict__ D, long long M, int H, long long o_stride,
                                                            long long do_stride) {
    constexpr int LPR = HD / 8;                       // lanes per row
    constexpr int ROWS_PER_BLOCK = 256 / LPR;
    const int sub = threadIdx.x % LPR;
    const long long total = M * H;
    const long long stride = (long long)gridDim.x * ROWS_PER_BLOCK;
    for (long long base = (long long)blockIdx.x * ROWS_PER_BLOCK + threadIdx.x / LPR; base < total; base += 4 * stride) {
        uint4 a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long it = base + u * stride;
            if (it < total) {
                const long long m = it / H;
                const int h = int(it - m * H);
                a[u] = *reinterpret_cast<const uint4*>(o + m * o_stride + h * HD + sub * 8);
                b[u] = *reinterpret_cast<const uint4*>(dout + m * do_stride + h * HD + sub * 8);
            } else {
                a[u] = make_uint4(0, 0, 0, 0);
                b[u] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float2 a0 = unpack_bf16x2(a[u].x), a1 = unpack_bf16x2(a[u].y), a2 = unpack_bf16x2(a[u].z), a3 = unpack_bf16x2(a[u].w);
            const float2 b0 = unpack_bf16x2(b[u].x), b1 = unpack_bf16x2(b[u].y), b2 = unpack_bf16x2(b[u].z), b3 = unpack_bf16x2(b[u].w);
            float acc = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
#pragma unroll
            for (int off = LPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            const long long it = base + u * stride;
            if (sub == 0 && it < total) {
                const long long m = it / H;
                const int h = int(it - m * H);
                D[(long long)h * M + m] = acc;
            }
        }
    }
}

// dq (fp32 accumulator, [M, H*HD]) -> inverse RoPE -> bf16 q columns of dqkv. In the same pass the
// k columns of dqkv (already bf16, written by the backward kernel) get their inverse RoPE in place.
__global__ void attn_bwd_finish_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv,
                                       const float* __restrict__ table, long long M, int T, int H, int KV, int HD,
                                       long long stride, int apply_rope) {
    const int vph = HD / 8;
    const long long total = M * (H + KV) * vph;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int v = int(i % vph);
        const long long t = i / vph;
        const int h = int(t % (H + KV));
        const long long m = t / (H + KV);
        float f[8];
        __nv_bfloat16* dst = dqkv + m * stride + h * HD + v * 8;
        if (h < H) {
            const float4* src = reinterpret_cast<const float4*>(dq_acc + m * (H * HD) + h * HD + v * 8);
            const float4 a = src[0], b = src[1];
            f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
        } else {
            const uint4 u = *reinterpret_cast<const uint4*>(dst);
            float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
            f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = cc.x; f[5] = cc.y; f[6] = d.x; f[7] = d.y;
        }
        float o[8];
        if (apply_rope) {
            const int pos = int(m % T);
            const float4* cs = reinterpret_cast<const float4*>(table + ((long long)pos * (HD / 2) + v * 4) * 2);
            const float4 c0 = cs[0], c1 = cs[1];
            const float co[4] = {c0.x, c0.z, c1.x, c1.z};
            const float si[4] = {-c0.y, -c0.w, -c1.y, -c1.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                o[2 * k] = f[2 * k] * co[k] - f[2 * k + 1] * si[k];
                o[2 * k + 1] = f[2 * k] * si[k] + f[2 * k + 1] * co[k];
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = f[k];
        }
        uint4 u;
        u.x = pack_bf16x2(o[0], o[1]); u.y = pack_bf16x2(o[2], o[3]); u.z = pack_bf16x2(o[4], o[5]); u.w = pack_bf16x2(o[6], o[7]);
        *reinterpret_cast<uint4*>(dst) = u;
    }
}

// nq[kv_tile] = number of query tiles that can see the kv tile: the diagonal tile plus every later tile whose first
// row's sequence starts at or before the tile's last kv row (seq_start is non-decreasing). One warp per kv tile, 32
// candidate tiles per step (one load latency per 32 tiles instead of one per tile). Also zeroes the work counter.
__global__ void attn_bwd_span_kernel(const int* __restrict__ seq_start, int n_tiles, int* __restrict__ nq, int* counter) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *counter = 0;
    const int kv_tile = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (kv_tile >= n_tiles) return;
    const int kv_last = kv_tile * 128 + 127;
    int n_q = 1;
    for (int t0 = kv_tile + 1; t0 < n_tiles; t0 += 32) {
        const int t = t0 + lane;
        const bool sees = t < n_tiles && seq_start[t * 128] <= kv_last;
        const uint32_t m = __ballot_sync(0xffffffffu, sees);
        const int run = __ffs(~m) - 1;          // leading run of visible tiles (m == all ones: ffs(0) - 1 = -1)
        if (run >= 0) { n_q += run; break; }
        n_q += 32;
    }
    if (lane == 0) nq[kv_tile] = n_q;
}

int sm_count();
int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);
int make_tmap_f32_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t box_inner, uint32_t box_outer);

template <int HD>
static int launch_attn_bwd(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tdq, const AttnBwdParams& p,
                           cudaStream_t st) {
    using Cfg = AttnBwdCfg<HD>;
    auto kern = attn_bwd_kernel<HD>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return -20;
        configured = true;
    }
    const int grid = p.n_items < sm_count() ? p.n_items : sm_count();     // one CTA per SM draws items until none are left
    attn_bwd_span_kernel<<<(p.n_tiles * 32 + 255) / 256, 256, 0, st>>>(p.seq_start, p.n_tiles, p.nq, p.counter);
    kern<<<grid, 512, Cfg::SMEM_BYTES, st>>>(tq, tdo, tdq, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

}  // namespace pb

// dq_acc: fp32 [M, H*HD] scratch (zeroed here); D: fp32 [H, M] scratch, computed here from o and dout unless o is
// null (then the caller has already filled it). Writes all of dqkv.
// rope_table != null: the inverse rotation is applied to dq and dk on the way out (position = row % T).
// tile_scratch: >= ceil(M / 128) + 1 ints of device scratch (query-tile count of every kv tile and the work counter).
extern "C" int pb_attn_bwd(const void* qkv, const void* o, const void* dout, const float* lse2, const int* seq_start,
                           void* dqkv, float* dq_acc, float* D, const float* rope_table, int T, int M, int H, int KV, int HD,
                           long long qkv_stride, long long o_stride, long long do_stride, long long dqkv_stride, float scale,
                           int* tile_scratch, int* status, void* stream) {
    using namespace pb;
    if (HD != 64 && HD != 128) return -1;
    if (H % KV) return -1;
    if ((qkv_stride % 8) || (o_stride % 8) || (do_stride % 8) || (dqkv_stride % 8)) return -2;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    CUtensorMap tq, tdo, tdq;
    int rc = make_tmap_bf16_2d(&tq, qkv, uint64_t(H + 2 * KV) * HD, M, qkv_stride, 64, 128);
    if (rc) return rc;
    rc = make_tmap_bf16_2d(&tdo, dout, uint64_t(H) * HD, M, do_stride, 64, 128);
    if (rc) return rc;
    rc = make_tmap_f32_2d(&tdq, dq_acc, uint64_t(H) * HD, M, uint64_t(H) * HD, 32, 32);
    if (rc) return rc;
    if (cudaMemsetAsync(dq_acc, 0, size_t(M) * H * HD * sizeof(float), st) != cudaSuccess) return -40;
    if (o) {   // o == null: the caller already filled D
        const long long rows = (long long)M * H;
        const int rows_per_block = 256 / (HD / 8);
        long long blocks = (rows + 4LL * rows_per_block - 1) / (4LL * rows_per_block);
        if (blocks < 1) blocks = 1;
        if (HD == 64)
            attn_bwd_prep_kernel<64><<<unsigned(blocks), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, D, M, H,
                                                                         o_stride, do_stride);
        else
            attn_bwd_prep_kernel<128><<<unsigned(blocks), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, D, M, H,
                                                                          o_stride, do_stride);
    }
    AttnBwdParams p;
    p.M = M; p.H = H; p.KV = KV; p.n_tiles = (M + 127) / 128; p.seq_start = seq_start; p.lse2 = lse2; p.D = D;
    p.dq_acc = dq_acc; p.dqkv = reinterpret_cast<__nv_bfloat16*>(dqkv); p.dqkv_stride = dqkv_stride;
    p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    if (tile_scratch == nullptr) return -3;
    p.nq = tile_scratch; p.counter = tile_scratch + p.n_tiles; p.n_items = p.n_tiles * KV;
    rc = HD == 64 ? launch_attn_bwd<64>(tq, tdo, tdq, p, st) : launch_attn_bwd<128>(tq, tdo, tdq, p, st);
    if (rc) return rc;
    const long long total = (long long)M * (H + KV) * (HD / 8);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    attn_bwd_finish_kernel<<<unsigned(blocks), 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dqkv, rope_table, M, T, H, KV, HD, dqkv_stride,
                                                              rope_table != nullptr);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}
