// Pieces shared by the single-CTA and the CTA-pair GEMM kernels: parameters, tile constants and
// the store of one 32-column accumulator chunk (one thread = one output row).
#pragma once
#include "common.cuh"

namespace pb {

constexpr int BM = 128;
constexpr int BK = 64;            // 64 bf16 = 128 B = one swizzle row
constexpr int UMMA_K = 16;

struct GemmParams {
    int M, N, K;
    void* C;         // output, bf16 or fp32
    const void* R;   // optional addend with the layout/dtype of C (may alias C)
    long long ldc, ldr;
    int out_fp32;
    int* status;
    int num_tiles, tiles_n;
    // CTA-pair kernel: tiles are numbered in bands of group_m tile rows (see gemm_tile_mn); tiles_m = rows of tiles
    int tiles_m, group_m;
    int tn_rot;      // tile columns are visited starting at this one (all-gather GEMM: the n-block fetched first)
    // split-K: work item w = slice * num_tiles + tile; slice s covers k-blocks [s * kb_per_split, ...) and
    // stores its fp32 partial tile at C + s * split_stride elements (plain direct-store epilogue only)
    int num_items, kb_per_split;
    long long split_stride;
    // fused epilogues of the CTA-pair kernel (GEMM_EPI_*); 0 = plain store
    int epi, epi_i0, epi_i1, epi_i2;
    int staged;      // plain / RoPE epilogue: 1 = stage the bf16 tile in shared memory and store it with TMA
    void* aux;
    long long ldaux;
    void* aux2;
};

// Output tile number -> tile row and tile column. Tiles are numbered in bands of group_m tile rows, down the rows of
// a band first, so that the tiles in flight at one time (one per CTA pair, consecutive numbers) cover a near-square
// block of the output and share their operand row blocks through L2: a band of 8 rows lets 74 pairs touch 8 + 10
// operand blocks per k-step instead of 1 + 74. group_m <= 1: plain row-major numbering.
__device__ __forceinline__ void gemm_tile_mn(const GemmParams& p, int tile, int& tm, int& tn) {
    if (p.group_m <= 1) {
        tm = tile / p.tiles_n;
        tn = tile % p.tiles_n;
        if (p.tn_rot) tn = (tn + p.tn_rot) % p.tiles_n;
        return;
    }
    const int band = p.group_m * p.tiles_n;
    const int g = tile / band;
    const int first = g * p.group_m;
    const int rows = p.tiles_m - first < p.group_m ? p.tiles_m - first : p.group_m;
    const int r = tile - g * band;
    tm = first + r % rows;
    tn = r / rows;
    if (p.tn_rot) tn = (tn + p.tn_rot) % p.tiles_n;
}

// Epilogues fused into the CTA-pair GEMM:
//  SWIGLU : B = [w1; w3] ([2F, K], F = epi_i0). A tile is 128 gate columns AND the matching 128 up
//           columns (the two CTAs of the pair load those two row ranges of B), so one thread holds
//           gate and up of the same feature: it stores both into C = h13 [M, 2F] and
//           silu(gate) * up into aux = act [M, F].
//  ROPE   : rotary embedding of the leading epi_i1 output columns (heads of epi_i2 columns,
//           position = row % epi_i0, aux = fp32 table [T, hd/2, 2] of (cos, sin)) before the store.
//  DSWIGLU: the product is d(act) [M, F = epi_i0]; aux = h13 [M, 2F] holds gate | up and is overwritten
//           in place with d(gate) | d(up). Nothing is written to C.
//  ROWDOT : besides the plain bf16 store of C, aux2[(col / epi_i0) * M + row] = sum over the epi_i0 (= 64) columns of
//           one head of C[row, col] * aux[row, col] (fp32 accumulator values times a bf16 matrix of C's shape):
//           the dO . O row sums that the attention backward needs, taken where dO is produced.
//  ADD    : C = product + aux (bf16, same shape; aux may be C itself): the residual / accumulate form of the staged
//           epilogue; the addend tiles arrive by TMA one round ahead.
constexpr int GEMM_EPI_NONE = 0, GEMM_EPI_SWIGLU = 1, GEMM_EPI_ROPE = 2, GEMM_EPI_DSWIGLU = 3, GEMM_EPI_ROWDOT = 4, GEMM_EPI_ADD = 5;

__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const float (&f)[32]) {
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        uint4 o;
        o.x = pack_bf16x2(f[j], f[j + 1]); o.y = pack_bf16x2(f[j + 2], f[j + 3]);
        o.z = pack_bf16x2(f[j + 4], f[j + 5]); o.w = pack_bf16x2(f[j + 6], f[j + 7]);
        *reinterpret_cast<uint4*>(dst + j) = o;
    }
}
// v: 32 consecutive fp32 accumulator columns of output row `row`, starting at column `col`.
__device__ __forceinline__ void gemm_store_chunk(const GemmParams& p, const uint32_t (&v)[32], int row, int col) {
    if (row >= p.M || col >= p.N) return;
    const int ncols = min(32, p.N - col);
    if (p.out_fp32) {
        float* dst = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col;
        const float* add = p.R ? reinterpret_cast<const float*>(p.R) + (long long)row * p.ldr + col : nullptr;
        if (ncols == 32) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                float4 o = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                if (add) {
                    float4 a = *reinterpret_cast<const float4*>(add + j);
                    o.x += a.x; o.y += a.y; o.z += a.z; o.w += a.w;
                }
                *reinterpret_cast<float4*>(dst + j) = o;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols) dst[j] = __uint_as_float(v[j]) + (add ? add[j] : 0.f);
        }
    } else {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col;
        const __nv_bfloat16* add = p.R ? reinterpret_cast<const __nv_bfloat16*>(p.R) + (long long)row * p.ldr + col : nullptr;
        if (ncols == 32) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                float f[8];
#pragma unroll
                for (int t = 0; t < 8; ++t) f[t] = __uint_as_float(v[j + t]);
                if (add) {
                    uint4 a = *reinterpret_cast<const uint4*>(add + j);
                    float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
                    f[0] += a0.x; f[1] += a0.y; f[2] += a1.x; f[3] += a1.y;
                    f[4] += a2.x; f[5] += a2.y; f[6] += a3.x; f[7] += a3.y;
                }
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(dst + j) = o;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols) dst[j] = __float2bfloat16(__uint_as_float(v[j]) + (add ? __bfloat162float(add[j]) : 0.f));
        }
    }
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                      uint32_t box_outer);
int sm_count();

}  // namespace pb
