// RMSNorm backward kernels, shared by the regular entry point (elementwise.cu) and the
// allocation-free one (elementwise_noalloc.cu).
#pragma once
#include "common.cuh"

namespace pb {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 u;
    u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
    u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(p) = u;
}

// ----------------------------------------------------------------------------
// RMSNorm backward. WPR warps share a row (one warp per row for N <= 1024, so that nothing of a row has to
// wait for another warp; two or four for wider rows, whose registers one warp cannot hold); each lane owns
// columns lane*8 + 256*j of its warp's CPW = NCH / WPR chunks.
//   xhat = x*rstd ; g = dy*w ; dx = (g - xhat * mean(g*xhat)) * rstd (+ dres)
//   dw  += dy * xhat  (per-CTA partials in fp32, reduced by a second kernel in fixed order)
// NCH = N / 256 column chunks per row.
// ----------------------------------------------------------------------------
template <int NCH, int WPR = 1>
__global__ void __launch_bounds__(256, 2) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          const float* __restrict__ rstd,
                                                          const __nv_bfloat16* __restrict__ dy,
                                                          const __nv_bfloat16* __restrict__ dres,
                                                          __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial,
                                                          int M) {
    constexpr int N = NCH * 256;
    constexpr int CPW = NCH / WPR;            // chunks per warp
    constexpr int RPI = 8 / WPR;              // rows per CTA iteration
    static_assert(NCH % WPR == 0 && 8 % WPR == 0 && CPW <= 4, "row split");
    __shared__ float red[8][32 * 8 + 1];
    __shared__ float s_w[N];
    __shared__ float s_dot[2][8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = warp % WPR, rslot = warp / WPR;
    const int col0 = sub * CPW * 256 + lane * 8;
    for (int c = threadIdx.x; c < N; c += blockDim.x) s_w[c] = __bfloat162float(w[c]);
    float dwacc[CPW][8];
#pragma unroll
    for (int j = 0; j < CPW; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) dwacc[j][i] = 0.f;
    __syncthreads();
    int it = 0;
    // (with several warps per row the whole CTA loops together because of the barrier below: warps past the
    // last row run empty iterations)
    for (long long base = (long long)blockIdx.x * RPI; WPR == 1 ? base + rslot < M : base < M;
         base += (long long)gridDim.x * RPI, ++it) {
        const long long row = base + rslot;
        const bool live = WPR == 1 ? true : row < M;
        // issue every load of the row before the first use, so one memory latency covers all of them
        uint4 ux[CPW], uy[CPW], ur[CPW];
        float r = 0.f;
        if (live) {
#pragma unroll
            for (int j = 0; j < CPW; ++j) {
                ux[j] = *reinterpret_cast<const uint4*>(x + row * N + col0 + j * 256);
                uy[j] = *reinterpret_cast<const uint4*>(dy + row * N + col0 + j * 256);
                if (dres) ur[j] = *reinterpret_cast<const uint4*>(dres + row * N + col0 + j * 256);
            }
            r = rstd[row];
        } else {
#pragma unroll
            for (int j = 0; j < CPW; ++j) ux[j] = uy[j] = ur[j] = make_uint4(0, 0, 0, 0);
        }
        // pass 1 over the registers: the row's dot product and the dw terms; pass 2 recomputes xhat and g from the
        // packed words instead of keeping 2 x CPW x 8 floats alive across the reduction
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < CPW; ++j) {
            const uint32_t wx[4] = {ux[j].x, ux[j].y, ux[j].z, ux[j].w}, wy[4] = {uy[j].x, uy[j].y, uy[j].z, uy[j].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 fx = unpack_bf16x2(wx[i]), fy = unpack_bf16x2(wy[i]);
                const int c = col0 + j * 256 + 2 * i;
                const float xa = fx.x * r, xb = fx.y * r;
                dot += (fy.x * s_w[c]) * xa + (fy.y * s_w[c + 1]) * xb;
                dwacc[j][2 * i] += fy.x * xa;
                dwacc[j][2 * i + 1] += fy.y * xb;
            }
        }
        dot = warp_sum(dot);
        if constexpr (WPR > 1) {
            // the row's warps add their parts in warp order (double-buffered by iteration: one barrier per row)
            if (lane == 0) s_dot[it & 1][warp] = dot;
            __syncthreads();
            dot = 0.f;
#pragma unroll
            for (int k = 0; k < WPR; ++k) dot += s_dot[it & 1][rslot * WPR + k];
        }
        dot *= (1.f / N);
        if (live) {
#pragma unroll
            for (int j = 0; j < CPW; ++j) {
                const uint32_t wx[4] = {ux[j].x, ux[j].y, ux[j].z, ux[j].w}, wy[4] = {uy[j].x, uy[j].y, uy[j].z, uy[j].w};
                float o[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 fx = unpack_bf16x2(wx[i]), fy = unpack_bf16x2(wy[i]);
                    const int c = col0 + j * 256 + 2 * i;
                    o[2 * i] = (fy.x * s_w[c] - (fx.x * r) * dot) * r;
                    o[2 * i + 1] = (fy.y * s_w[c + 1] - (fx.y * r) * dot) * r;
                }
                if (dres) {
                    const uint32_t wr[4] = {ur[j].x, ur[j].y, ur[j].z, ur[j].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 fr = unpack_bf16x2(wr[i]);
                        o[2 * i] += fr.x;
                        o[2 * i + 1] += fr.y;
                    }
                }
                store8(dx + row * N + col0 + j * 256, o);
            }
        }
    }
    // fixed-order reduction of the per-warp dw accumulators across the CTA: for each chunk, the warps that
    // hold the same columns (same `sub`) are added in row-slot order by warp `sub`
    for (int j = 0; j < CPW; ++j) {
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; ++i) red[warp][lane * 8 + i] = dwacc[j][i];
        __syncthreads();
        if (warp < WPR) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float s = 0.f;
                for (int rs = 0; rs < RPI; ++rs) s += red[rs * WPR + warp][lane * 8 + i];
                dw_partial[(long long)blockIdx.x * N + warp * CPW * 256 + j * 256 + lane * 8 + i] = s;
            }
        }
    }
}

// dw[c] (+)= sum_b partial[b, c]; output bf16 or fp32. One block = 32 columns x 8 row groups: every thread
// sums the rows b = g, g + 8, ... of its column with four loads in flight, the eight group sums are then
// added in a fixed order (deterministic for a given number of partial rows).
static __global__ void __launch_bounds__(256) colsum_partials_kernel(const float* __restrict__ partial, void* __restrict__ out,
                                                                     int nb, int N, int out_fp32, int accumulate) {
    __shared__ float red[8][33];
    const int cx = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cx;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (c < N) {
        int b = g;
        for (; b + 24 < nb; b += 32) {
            s0 += partial[(long long)b * N + c];
            s1 += partial[(long long)(b + 8) * N + c];
            s2 += partial[(long long)(b + 16) * N + c];
            s3 += partial[(long long)(b + 24) * N + c];
        }
        for (; b < nb; b += 8) s0 += partial[(long long)b * N + c];
    }
    red[g][cx] = (s0 + s1) + (s2 + s3);
    __syncthreads();
    if (g == 0 && c < N) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) s += red[k][cx];
        if (out_fp32) {
            float* o = reinterpret_cast<float*>(out);
            o[c] = accumulate ? o[c] + s : s;
        } else {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
            o[c] = __float2bfloat16(accumulate ? __bfloat162float(o[c]) + s : s);
        }
    }
}

}  // namespace pb
