// Causal / document-masked GQA flash attention forward for sm_100a on tcgen05 + TMEM + TMA.
//
// Input is the fused, already rotated projection buffer qkv[M, (H + 2*KV) * HD]:
// q head h at column h*HD, k head g at (H + g)*HD, v head g at (H + KV + g)*HD.
// The M rows are a packed token stream; seq_start[m] is the first row query m may attend to
// (start of its batch row or, with sequence packing, of its document), and m itself is the
// last (causal). This replaces repeat_kv + FlexAttention/SDPA of the reference
// (models/llama/model.py:147-156, 168-198, 282-302): KV heads are indexed, never expanded,
// and the document mask comes from seq_start, not from a BlockMask.
//
// One CTA = one 128-row query tile of one head, 256 threads in two warpgroups: warp 0 TMA producer, warp 1 MMA
// issuer (owns TMEM), warps 2-3 only hold the first warpgroup together, warps 4-7 softmax (one thread per query
// row: row max / sum are thread-local). At head size 64, where two CTAs share an SM, the first warpgroup gives
// registers up (setmaxnreg) so that a softmax thread can hold its 128-wide score row without spilling.
//   S = Q K^T            -> TMEM [128 x 128] fp32
//   P = exp2(S*c - m*c)  -> bf16 pairs in TMEM (tcgen05.st), read by the PV MMA as its A operand
//   O  += P V            -> TMEM [128 x HD] fp32, accumulated by the MMA across KV tiles; rows are
//                           rescaled in TMEM only when their running maximum grows by > 2^8
// Outputs: o[M, H*HD] bf16 and lse2[H, M] = log2-sum-exp of the scaled scores (log2 units).
#include "common.cuh"

namespace pb {

struct AttnFwdParams {
    int M, H, KV;
    const int* seq_start;
    __nv_bfloat16* O;
    long long o_stride;
    float* lse2;
    float scale_log2;   // softmax scale * log2(e)
    int* status;
};

template <int HD>
struct AttnFwdCfg {
    static constexpr int TILE_BYTES = 128 * HD * 2;          // one Q / K / V tile
    static constexpr int KV_STAGES = 2;
    // two CTAs of the HD=64 variant must fit one SM, so there is no alignment slack: the kernel
    // checks that the dynamic shared window is 1024-byte aligned and reports an error otherwise
    static constexpr int SMEM_BYTES = TILE_BYTES * (1 + 2 * KV_STAGES) + 128;
    // TMEM columns: S (fp32) 0..127, O (fp32) 128..128+HD, P (bf16 pairs, A operand of the PV MMA) next 64
    static constexpr int T_P = 128 + HD;
    static constexpr int TMEM_COLS = (HD == 64) ? 256 : 512;
};

__device__ __forceinline__ void fwd_reg_dealloc_40() { asm volatile("setmaxnreg.dec.sync.aligned.u32 40;"); }
__device__ __forceinline__ void fwd_reg_alloc_216() { asm volatile("setmaxnreg.inc.sync.aligned.u32 216;"); }

template <int HD>
__global__ void __launch_bounds__(256, (HD == 64 ? 2 : 1))
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm, const AttnFwdParams p) {
    using Cfg = AttnFwdCfg<HD>;
    constexpr int NB = HD / 64;   // 64-column swizzle blocks per tile
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    if (base & 1023u) {
        if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, PB_ERR_TIMEOUT_MISC | 0x80);
        return;
    }
    uint8_t* gen = smem_raw;
    const uint32_t sQ = base;
    const uint32_t sK = sQ + Cfg::TILE_BYTES;                           // [2]
    const uint32_t sV = sK + Cfg::KV_STAGES * Cfg::TILE_BYTES;           // [2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(gen + Cfg::TILE_BYTES * (1 + 2 * Cfg::KV_STAGES));
    const uint32_t bar_q = smem_u32(bars);
    const uint32_t bar_kfull = bar_q + 8;        // [2]
    const uint32_t bar_vfull = bar_kfull + 16;   // [2]
    const uint32_t bar_kvempty = bar_vfull + 16; // [2]
    const uint32_t bar_sfull = bar_kvempty + 16;
    const uint32_t bar_pfull = bar_sfull + 8;
    const uint32_t bar_ofull = bar_pfull + 8;
    const uint32_t bar_sfree = bar_ofull + 8;    // softmax warps hold S_j in registers: S TMEM may be overwritten
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_tile = gridDim.x - 1 - blockIdx.x;   // heaviest (latest) tiles first
    const int head = blockIdx.y;
    const int kvh = head / (p.H / p.KV);
    const int q0 = q_tile * 128;

    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_kfull + 8 * s, 1);
            mbar_init(bar_vfull + 8 * s, 1);
            mbar_init(bar_kvempty + 8 * s, 1);
        }
        mbar_init(bar_sfull, 1);
        mbar_init(bar_pfull, 4);
        mbar_init(bar_ofull, 1);
        mbar_init(bar_sfree, 4);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tm);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tS = tmem_base, tO = tmem_base + 128, tP = tmem_base + Cfg::T_P;

    // kv tile range: from the tile holding the first row's sequence start up to the diagonal
    const int first_start = p.seq_start[min(q0, p.M - 1)];
    const int kv_lo = first_start / 128;
    const int kv_hi = q_tile;                      // inclusive
    const int n_kv = kv_hi - kv_lo + 1;

    // head size 64: 2 CTAs x (128 x 40 + 128 x 216) registers = the SM's 64 K
    if (warp < 4) {
        if (HD == 64) fwd_reg_dealloc_40();
        if (warp == 0) {
            // ------------------------------ TMA producer ------------------------------
            if (lane == 0) {
                mbar_expect_tx(bar_q, Cfg::TILE_BYTES);
#pragma unroll
                for (int b = 0; b < NB; ++b) tma_load_2d(sQ + b * 16384, &tm, bar_q, head * HD + 64 * b, q0);
            }
            bool ok = true;
            for (int j = 0; j < n_kv && ok; ++j) {
                const int st = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                ok = mbar_wait(bar_kvempty + 8 * st, ph ^ 1, abort_flag, p.status, PB_ERR_TIMEOUT_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (lane == 0) {
                    const int kv0 = (kv_lo + j) * 128;
                    mbar_expect_tx(bar_kfull + 8 * st, Cfg::TILE_BYTES);
#pragma unroll
                    for (int b = 0; b < NB; ++b)
                        tma_load_2d(sK + st * Cfg::TILE_BYTES + b * 16384, &tm, bar_kfull + 8 * st, (p.H + kvh) * HD + 64 * b, kv0);
                    mbar_expect_tx(bar_vfull + 8 * st, Cfg::TILE_BYTES);
#pragma unroll
                    for (int b = 0; b < NB; ++b)
                        tma_load_2d(sV + st * Cfg::TILE_BYTES + b * 16384, &tm, bar_vfull + 8 * st, (p.H + p.KV + kvh) * HD + 64 * b, kv0);
                }
                __syncwarp();
            }
            if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(10000);
        } else if (warp == 1) {
            // ------------------------------ MMA issuer ------------------------------
            constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t idesc_o = umma_idesc_bf16(128, HD, 0, 1);
            auto issue_s = [&](int st) {
                const uint32_t kb = sK + st * Cfg::TILE_BYTES;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
                    umma_f16_ss(tS, umma_smem_desc(sQ + off, 16, 1024), umma_smem_desc(kb + off, 16, 1024), idesc_s, k ? 1u : 0u);
                }
                umma_commit(bar_sfull);
            };
            bool ok = mbar_wait(bar_q, 0, abort_flag, p.status, PB_ERR_TIMEOUT_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                ok = mbar_wait(bar_kfull, 0, abort_flag, p.status, PB_ERR_TIMEOUT_FULL);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
                tc_fence_after();
                if (lane == 0) issue_s(0);
                __syncwarp();
            }
            for (int j = 0; j < n_kv && ok; ++j) {
                const int st = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                if (j + 1 < n_kv) {
                    // S_{j+1} is issued as soon as the softmax warps have pulled S_j into registers, so the
                    // tensor core computes it while they do the exponentials of tile j
                    const int st1 = (j + 1) & 1;
                    const uint32_t ph1 = ((j + 1) >> 1) & 1;
                    ok = mbar_wait(bar_sfree, j & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    ok = mbar_wait(bar_kfull + 8 * st1, ph1, abort_flag, p.status, PB_ERR_TIMEOUT_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    if (lane == 0) issue_s(st1);
                    __syncwarp();
                }
                ok = mbar_wait(bar_pfull, j & 1, abort_flag, p.status, PB_ERR_TIMEOUT_MISC);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ok = mbar_wait(bar_vfull + 8 * st, ph, abort_flag, p.status, PB_ERR_TIMEOUT_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t vb = sV + st * Cfg::TILE_BYTES;
#pragma unroll
                    for (int k = 0; k < 8; ++k) {   // 128 kv rows, 16 per step
                        // A = P straight from tensor memory: 16 bf16 of every row = 8 columns per K-step
                        const uint64_t db = umma_smem_desc(vb + k * 2048, 16384, 1024);
                        umma_f16_ts(tO, tP + k * 8, db, idesc_o, (j | k) ? 1u : 0u);   // O accumulates over all kv tiles
                    }
                    umma_commit(bar_ofull);
                    umma_commit(bar_kvempty + 8 * st);
                }
                __syncwarp();
            }
        }
    } else {
        if (HD == 64) fwd_reg_alloc_216();
        // ------------------------------ softmax warps ------------------------------
        // One thread per query row. The whole 128-wide score row is pulled from TMEM in one go and
        // stays in registers; O lives in TMEM (the PV MMA accumulates into it) and is rescaled only
        // when a row's running maximum grows by more than 2^8 -- until then exponentials use the
        // older maximum, which is exact after the final division by the row sum.
        const int quad = warp & 3;
        const int r = quad * 32 + lane;           // row within the tile == TMEM lane
        const int row = q0 + r;
        const uint32_t lane_off = uint32_t(quad * 32) << 16;
        const int my_start = p.seq_start[min(row, p.M - 1)];
        const int tile_last_start = p.seq_start[min(q0 + 127, p.M - 1)];
        const float c = p.scale_log2;
        float m_used = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kv && ok; ++j) {
            const int kv0 = (kv_lo + j) * 128;
            ok = mbar_wait(bar_sfull, j & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            uint32_t v[4][32];
#pragma unroll
            for (int q = 0; q < 4; ++q) tmem_ld32(tS + lane_off + 32 * q, v[q]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sfree);
            const bool need_mask = (kv0 + 127 > q0) || (kv0 < tile_last_start);
            // row maximum: 3-input max over four independent chains
            if (need_mask) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int s = kv0 + 32 * q + i;
                        if (!(s <= row && s >= my_start)) v[q][i] = 0xff800000u;      // -inf
                    }
            }
            float mxp[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int i = 0; i < 32; i += 2)
                    mxp[(i >> 1) & 3] = max3(mxp[(i >> 1) & 3], __uint_as_float(v[q][i]), __uint_as_float(v[q][i + 1]));
            const float mx = fmaxf(fmaxf(mxp[0], mxp[1]), fmaxf(mxp[2], mxp[3]));
            bool o_done = (j == 0);   // PV of the previous tile has retired (P and O may be touched)
            const bool grow = (mx != -INFINITY) && (m_used == -INFINITY || (mx - m_used) * c > 8.f);
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? fmaxf(m_used, mx) : m_used;
                const float alpha = (m_used == -INFINITY) ? 0.f : exp2f((m_used - m_new) * c);
                if (j > 0) {      // O of the previous tiles exists: wait until its last PV retired, then rescale the row
                    ok = mbar_wait(bar_ofull, (j - 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    o_done = true;
                    tc_fence_after();
#pragma unroll
                    for (int cidx = 0; cidx < HD; cidx += 32) {
                        uint32_t o[32];
                        tmem_ld32(tO + lane_off + cidx, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(tO + lane_off + cidx, o);
                    }
                    tmem_st_wait();
                }
                l_run *= alpha;
                m_used = m_new;
            }
            const float m_sub = (m_used == -INFINITY) ? 0.f : m_used * c;
            if (!o_done) {   // the PV MMA of the previous tile still reads P from tensor memory until it retires
                ok = mbar_wait(bar_ofull, (j - 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
            }
            // P = exp2(S*c - m*c): the scale-and-shift and the row sum run on packed fp32 pairs (one f32x2
            // instruction per two scores), the exponentials on the special-function unit (16 per clock per SM
            // whether packed or not, so they are taken in fp32, one per score)
            const unsigned long long cc = f32x2_pack(c, c), nm = f32x2_pack(-m_sub, -m_sub);
            unsigned long long rs2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t pw[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const unsigned long long x2 =
                        f32x2_fma(f32x2_pack(__uint_as_float(v[q][2 * i]), __uint_as_float(v[q][2 * i + 1])), cc, nm);
                    float x0, x1;
                    f32x2_unpack(x2, x0, x1);
                    const float e0 = ex2_approx(x0), e1 = ex2_approx(x1);      // masked entries are -inf -> 0
                    pw[i] = pack_bf16x2(e0, e1);
                    rs2[i & 3] = f32x2_add(rs2[i & 3], f32x2_pack(e0, e1));
                }
                tmem_st16(tP + lane_off + 16 * q, pw);   // 32 kv columns = 16 packed words of this row
            }
            {
                float a0, a1;
                f32x2_unpack(f32x2_add(f32x2_add(rs2[0], rs2[1]), f32x2_add(rs2[2], rs2[3])), a0, a1);
                l_run += a0 + a1;
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_pfull);
        }
        if (ok) {
            ok = mbar_wait(bar_ofull, (n_kv - 1) & 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            __nv_bfloat16* dst = p.O + (long long)row * p.o_stride + head * HD;
#pragma unroll
            for (int cidx = 0; cidx < HD; cidx += 32) {
                uint32_t o[32];
                tmem_ld32(tO + lane_off + cidx, o);
                tmem_ld_wait();
                if (row < p.M) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 u;
                        u.x = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                        u.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                        u.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                        u.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + cidx + i) = u;
                    }
                }
            }
            if (row < p.M) p.lse2[(long long)head * p.M + row] = (l_run > 0.f) ? (m_used * c + log2f(l_run)) : -INFINITY;
            tc_fence_before();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

template <int HD>
static int launch_attn_fwd(const CUtensorMap& tm, const AttnFwdParams& p, cudaStream_t st) {
    using Cfg = AttnFwdCfg<HD>;
    auto kern = attn_fwd_kernel<HD>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return -20;
        configured = true;
    }
    dim3 grid((p.M + 127) / 128, p.H);
    kern<<<grid, 256, Cfg::SMEM_BYTES, st>>>(tm, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

}  // namespace pb

extern "C" int pb_attn_fwd(const void* qkv, const int* seq_start, void* o, float* lse2, int M, int H, int KV, int HD,
                           long long qkv_stride, long long o_stride, float scale, int* status, void* stream) {
    using namespace pb;
    if (HD != 64 && HD != 128) return -1;
    if (H % KV) return -1;
    if ((qkv_stride % 8) || (o_stride % 8) || (reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(o) & 15)) return -2;
    CUtensorMap tm;
    int rc = make_tmap_bf16_2d(&tm, qkv, uint64_t(H + 2 * KV) * HD, M, qkv_stride, 64, 128);
    if (rc) return rc;
    AttnFwdParams p;
    p.M = M; p.H = H; p.KV = KV; p.seq_start = seq_start; p.O = reinterpret_cast<__nv_bfloat16*>(o); p.o_stride = o_stride;
    p.lse2 = lse2; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    return HD == 64 ? launch_attn_fwd<64>(tm, p, st) : launch_attn_fwd<128>(tm, p, st);
}
