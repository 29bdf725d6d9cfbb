// Persistent, warp-specialised bf16 GEMM for sm_100a built directly on tcgen05.mma
// with TMEM accumulators and TMA-fed shared-memory stages.
//
//   C[M,N] = op(A)[M,K] * op(B)[N,K]^T  (+ R)        fp32 accumulate
//
// A may be stored K-major ([M,K] row-major) or M-major ([K,M] row-major); B may be
// stored K-major ([N,K] row-major, i.e. an nn.Linear weight) or N-major ([K,N]).
// The three layouts a Linear layer needs map to:
//   forward  y  = x  W^T : A=x  K-major, B=W  K-major
//   dgrad    dx = dy W   : A=dy K-major, B=W  N-major
//   wgrad    dW = dy^T x : A=dy M-major, B=x  N-major
// (replaces the cuBLAS calls behind nn.Linear in models/llama/model.py:227-230,336-341,461
//  of the reference).
//
// Roles inside a CTA (192 threads): warp 0 issues TMA loads, warp 1 issues the MMAs and
// owns the TMEM allocation, warps 2-5 drain the accumulator (tcgen05.ld) and write C.
// Two TMEM accumulators let the epilogue of tile i overlap the main loop of tile i+1.
// No cluster multicast is used: each CTA loads its own operand tiles.
#include "gemm_common.cuh"
#include <mutex>

namespace pb {

template <int BN>
struct GemmCfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (BN == 256) ? 4 : 6;
    static constexpr int TMEM_COLS = 2 * BN;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_tcgen05(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const GemmParams p) {
    using Cfg = GemmCfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // barrier block lives after the stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES);
    const uint32_t bar_full = smem_u32(bars);                  // [STAGES]
    const uint32_t bar_empty = bar_full + 8 * STAGES;          // [STAGES]
    const uint32_t bar_tfull = bar_empty + 8 * STAGES;         // [2]
    const uint32_t bar_tempty = bar_tfull + 16;                // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_kb = (p.K + BK - 1) / BK;

    if (warp == 0) {
        // ------------------------- TMA producer -------------------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
            const int m0 = (tile / p.tiles_n) * BM;
            const int n0 = (tile % p.tiles_n) * BN;
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, PB_ERR_TIMEOUT_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
                    const uint32_t sb = sa + Cfg::A_BYTES;
                    const uint32_t fb = bar_full + 8 * stage;
                    mbar_expect_tx(fb, Cfg::STAGE_BYTES);
                    const int k0 = kb * BK;
                    if constexpr (!A_MN) {
                        tma_load_2d(sa, &tmA, fb, k0, m0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &tmA, fb, m0 + 64 * j, k0);
                    }
                    if constexpr (!B_MN) {
                        tma_load_2d(sb, &tmB, fb, k0, n0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &tmB, fb, n0 + 64 * j, k0);
                    }
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
        if (!ok) {
            // give copies already in flight a bounded moment to land before teardown
            for (int i = 0; i < 64; ++i) __nanosleep(10000);
        }
    } else if (warp == 1) {
        // ------------------------- MMA issuer -------------------------
        constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
        int stage = 0;
        uint32_t phase = 0;
        int local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++local) {
            const int acc = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            ok = mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_EMPTY);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BN;
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, PB_ERR_TIMEOUT_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
                    const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        uint64_t da, db;
                        if constexpr (!A_MN) da = umma_smem_desc(sa + k * (UMMA_K * 2), 16, 1024);
                        else                 da = umma_smem_desc(sa + k * (UMMA_K * 128), BK * 128, 1024);
                        if constexpr (!B_MN) db = umma_smem_desc(sb + k * (UMMA_K * 2), 16, 1024);
                        else                 db = umma_smem_desc(sb + k * (UMMA_K * 128), BK * 128, 1024);
                        umma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(bar_empty + 8 * stage);   // smem slot reusable once these MMAs retire
                    if (kb == num_kb - 1) umma_commit(bar_tfull + 8 * acc);
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else {
        // ------------------------- epilogue (warps 2..5) -------------------------
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
        const int row_in_tile = quad * 32 + lane;
        int local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++local) {
            const int acc = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            const int m0 = (tile / p.tiles_n) * BM;
            const int n0 = (tile % p.tiles_n) * BN;
            ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, PB_ERR_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = m0 + row_in_tile;
            const uint32_t t_row = tmem_base + acc * BN + (uint32_t(quad * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t v[32];
                tmem_ld32(t_row + c, v);
                tmem_ld_wait();
                gemm_store_chunk(p, v, row, n0 + c);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ----------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(f);
    });
    return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows, row pitch ld elements.
int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return -10;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -(1000 + int(r));
}

// 2-D fp32 tensor map (used as the destination of bulk reduce-adds)
int make_tmap_f32_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t box_inner, uint32_t box_outer) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return -10;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {ld * 4};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -(1000 + int(r));
}

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    }
    return n;
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams p, int max_ctas, cudaStream_t st) {
    using Cfg = GemmCfg<BN>;
    auto kern = gemm_bf16_tcgen05<BN, A_MN, B_MN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return -20;
        configured = true;
    }
    const int tiles_m = (p.M + BM - 1) / BM;
    p.tiles_n = (p.N + BN - 1) / BN;
    p.num_tiles = tiles_m * p.tiles_n;
    int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
    if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
    kern<<<grid, 192, Cfg::SMEM_BYTES, st>>>(tmA, tmB, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

}  // namespace pb

// C[M,N] = op(A) op(B)^T (+R).  a_mn: A stored [K,M]; b_mn: B stored [K,N].
// lda/ldb/ldc/ldr are row pitches in elements. status: device int (0 = ok) or null.
// bn: 0 = choose, else 128 or 256. max_ctas: 0 = all SMs (lets a caller leave SMs to a
// concurrent communication kernel).
extern "C" int pb_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                            long long lda, long long ldb, long long ldc, long long ldr, int a_mn, int b_mn,
                            int out_fp32, int bn, int max_ctas, int* status, void* stream) {
    using namespace pb;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -1;
    const int vec = out_fp32 ? 4 : 8;
    if ((ldc % vec) || (R && (ldr % vec)) || (reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(R) & 15)) return -2;
    if (bn == 0) {
        // prefer the wide tile unless it leaves most SMs idle
        const long long t256 = (long long)((M + BM - 1) / BM) * ((N + 255) / 256);
        bn = (N <= 128 || (t256 < 2 * sm_count() && N % 256 != 0) || t256 < sm_count() / 2) ? 128 : 256;
    }
    CUtensorMap tmA, tmB;
    int rc;
    if (!a_mn) rc = make_tmap_bf16_2d(&tmA, A, K, M, lda, BK, BM);
    else       rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, 64, BK);
    if (rc) return rc;
    if (!b_mn) rc = make_tmap_bf16_2d(&tmB, B, K, N, ldb, BK, bn);
    else       rc = make_tmap_bf16_2d(&tmB, B, N, K, ldb, 64, BK);
    if (rc) return rc;
    GemmParams p{};
    p.M = M; p.N = N; p.K = K; p.C = C; p.R = R; p.ldc = ldc; p.ldr = ldr; p.out_fp32 = out_fp32; p.status = status;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define PB_DISPATCH(BN_)                                                                       \
    if (!a_mn && !b_mn) return launch_gemm<BN_, false, false>(tmA, tmB, p, max_ctas, st);      \
    if (!a_mn && b_mn)  return launch_gemm<BN_, false, true>(tmA, tmB, p, max_ctas, st);       \
    if (a_mn && !b_mn)  return launch_gemm<BN_, true, false>(tmA, tmB, p, max_ctas, st);       \
    return launch_gemm<BN_, true, true>(tmA, tmB, p, max_ctas, st);
    if (bn == 256) { PB_DISPATCH(256) }
    PB_DISPATCH(128)
#undef PB_DISPATCH
}
