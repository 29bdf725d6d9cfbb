// DiLoCo outer step on the GPU: pseudo-gradient, uint8 quantisation, all-reduce over NVLink peer
// memory with fp32 accumulation, and the Nesterov outer update — executed by kernels that read and
// write the peers' symmetric buffers directly.
//
// Reference path being replaced: per-parameter device->host copies, CPU subtraction, the C++ gloo
// ring with a CPU quantiser, torch CPU SGD, host->device copies (src/zeroband/diloco.py:77-144,
// 203-215; C/csrc/collectives.cpp:76-230; C/csrc/compression.cpp:9-125).
//
// Group = the W ranks that hold the same parameter shard in the W workers. NVSwitch gives uniform
// all-to-all bandwidth, so instead of a ring the exchange is direct:
//   stage A (local)   d = (outer - inner) / W   [0 for a "fake" joiner]; per 1 Mi-element chunk:
//                     sigma from the un-centred L2 norm, scale = 6 sigma / 256,
//                     q = clamp(round(d / scale) + 128), codebook[b] = mean of members of bin b
//                     -> q (uint8) and codebooks land in this rank's symmetric buffer
//   stage B (pull)    rank r owns chunks [r*C/W, (r+1)*C/W): sum over all ranks p of
//                     codebook_p[q_p[i]] in fp32 (fixed rank order), then quantise the reduced slice
//                     ONCE into this rank's second symmetric buffer
//   stage C (pull)    every rank reads every owner's reduced bytes + codebook, dequantises to g and
//                     applies  m = mu*m + g ; outer -= lr*(g + mu*m) ; inner = outer
// Values are quantised twice in total (reference: W-1 times plus a re-quantisation per all-gather
// hop), and all ranks decode the same bytes, so they end bit-identical. Quantiser semantics follow
// the reference (round half away from zero, empty bin -> 0). All reductions are fixed-order.
// Synchronisation between stages is the bounded epoch barrier of zero_comm.cu (launched by the
// host wrapper between the kernels); there is no multicast TMA and no library collective here.
#include "common.cuh"

namespace pb {

constexpr int DL_MAX_RANKS = 16;
constexpr int DL_CHUNK = 1 << 20;         // elements per quantisation chunk
constexpr int DL_BLOCKS_PER_CHUNK = 16;   // CTAs cooperating on one chunk
constexpr int DL_THREADS = 512;

struct DlPeers {
    int world, rank;
    const uint8_t* q[DL_MAX_RANKS];       // stage A bytes of every rank   [n]
    const float* lut[DL_MAX_RANKS];       // stage A codebooks             [chunks][256]
    const uint8_t* q2[DL_MAX_RANKS];      // stage B bytes (owner slices)  [n]
    const float* lut2[DL_MAX_RANKS];      // stage B codebooks             [chunks][256]
};

__device__ __forceinline__ float block_sum(float v, float* smem) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    if (threadIdx.x == 0) {
        for (int i = 0; i < (blockDim.x >> 5); ++i) t += smem[i];
        smem[0] = t;
    }
    __syncthreads();
    t = smem[0];
    __syncthreads();
    return t;
}

// ---- pass 1: per (chunk, block) partial sum of squares of the value to be quantised ----
// mode 0: value = (outer - inner) * inv_w, or outer * inv_w when inner is null (plain all-reduce input),
//         or 0 if fake ; mode 1: value = src[i] (already reduced)
template <int MODE>
__global__ void __launch_bounds__(DL_THREADS) dl_sumsq_kernel(const float* __restrict__ a, const float* __restrict__ b, float inv_w,
                                                              int fake, long long n, long long first_chunk,
                                                              float* __restrict__ partial) {
    __shared__ float red[32];
    const long long chunk = first_chunk + blockIdx.x / DL_BLOCKS_PER_CHUNK;
    const int sub = blockIdx.x % DL_BLOCKS_PER_CHUNK;
    const long long lo = chunk * DL_CHUNK, hi = min(n, lo + (long long)DL_CHUNK);
    float s = 0.f;
    const long long off = MODE == 0 ? 0 : first_chunk * DL_CHUNK;
    // chunk starts are multiples of 4 elements, so float4 loads are aligned whenever the base pointers are
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
    for (long long i = lo + (sub * DL_THREADS + threadIdx.x) * 4ll; i < hi; i += DL_BLOCKS_PER_CHUNK * DL_THREADS * 4ll) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (aligned && i + 3 < hi) {
            if (!(MODE == 0 && fake)) {
                const float4 x = *reinterpret_cast<const float4*>(a + i - off);
                v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
                if (MODE == 0) {
                    if (b) {
                        const float4 y = *reinterpret_cast<const float4*>(b + i);
                        v[0] -= y.x; v[1] -= y.y; v[2] -= y.z; v[3] -= y.w;
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) v[k] *= inv_w;
                }
            }
        } else {
            for (int k = 0; k < 4 && i + k < hi; ++k) {
                if (MODE == 0) v[k] = fake ? 0.f : (b ? a[i + k] - b[i + k] : a[i + k]) * inv_w;
                else v[k] = a[i + k - off];
            }
        }
        s += (v[0] * v[0] + v[1] * v[1]) + (v[2] * v[2] + v[3] * v[3]);
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__device__ __forceinline__ float dl_chunk_scale(const float* __restrict__ sumsq_partial, int cb, long long cnt) {
    float ss = 0.f;
    for (int k = 0; k < DL_BLOCKS_PER_CHUNK; ++k) ss += sumsq_partial[cb * DL_BLOCKS_PER_CHUNK + k];
    const float sigma = sqrtf(ss / float(cnt > 1 ? cnt - 1 : 1));
    float scale = 6.f * sigma / 256.f;
    if (!(scale > 0.f) || isinf(scale)) scale = 1.f;   // all-zero chunk (e.g. a fake pseudo-gradient)
    return scale;
}

constexpr float DL_FX = 1048576.f;   // 2^20: bin sums are kept in fixed point (units of scale / 2^20)

// ---- pass 2: quantise + per-block bin sums / counts (shared-memory privatised) ----
// Bin sums are accumulated as 64-bit fixed-point integers of v/scale, so the result does not depend
// on the order in which threads arrive (integer addition is associative): the codebook is
// bit-reproducible run to run. The rounding step (2^-20 of a bin width) is far below fp32 noise.
template <int MODE>
__global__ void __launch_bounds__(DL_THREADS) dl_quantize_kernel(const float* __restrict__ a, const float* __restrict__ b, float inv_w,
                                                                 int fake, long long n, long long first_chunk,
                                                                 const float* __restrict__ sumsq_partial, uint8_t* __restrict__ q,
                                                                 long long* __restrict__ bin_sum, unsigned* __restrict__ bin_cnt) {
    // One shared-memory atomic per element: an inner bin b holds (count << 40) | sum of the fixed-point
    // offsets of its values from the bin's lower edge (b - 128.5), which lie in [0, 2^20]; at most 65536
    // elements of a chunk reach one block, so neither field can overflow. The two clamping end bins take
    // values from an unbounded range and keep an exact 64-bit sum and a count of their own.
    constexpr int COPIES = 8;                       // histogram copies: two warps share one
    __shared__ unsigned long long s_sum[COPIES][256];
    __shared__ unsigned long long s_edge_sum[2];
    __shared__ unsigned s_edge_cnt[2];
    const int cb = blockIdx.x / DL_BLOCKS_PER_CHUNK;
    const long long chunk = first_chunk + cb;
    const int sub = blockIdx.x % DL_BLOCKS_PER_CHUNK;
    const long long lo = chunk * DL_CHUNK, hi = min(n, lo + (long long)DL_CHUNK);
    for (int i = threadIdx.x; i < COPIES * 256; i += DL_THREADS) (&s_sum[0][0])[i] = 0ull;
    if (threadIdx.x < 2) { s_edge_sum[threadIdx.x] = 0ull; s_edge_cnt[threadIdx.x] = 0u; }
    const float inv_scale = 1.f / dl_chunk_scale(sumsq_partial, cb, hi - lo);
    __syncthreads();
    unsigned long long* my_sum = s_sum[(threadIdx.x >> 6) % COPIES];
    const long long off = MODE == 0 ? 0 : first_chunk * DL_CHUNK;
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0;
    for (long long i = lo + (sub * DL_THREADS + threadIdx.x) * 4ll; i < hi; i += DL_BLOCKS_PER_CHUNK * DL_THREADS * 4ll) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        const bool full = aligned && i + 3 < hi;
        if (full) {
            if (!(MODE == 0 && fake)) {
                const float4 x = *reinterpret_cast<const float4*>(a + i - off);
                v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
                if (MODE == 0) {
                    if (b) {
                        const float4 y = *reinterpret_cast<const float4*>(b + i);
                        v[0] -= y.x; v[1] -= y.y; v[2] -= y.z; v[3] -= y.w;
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) v[k] *= inv_w;
                }
            }
        } else {
            for (int k = 0; k < 4 && i + k < hi; ++k) {
                if (MODE == 0) v[k] = fake ? 0.f : (b ? a[i + k] - b[i + k] : a[i + k]) * inv_w;
                else v[k] = a[i + k - off];
            }
        }
        uint32_t packed = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (full || i + k < hi) {
                const float t = v[k] * inv_scale;
                int qi = __float2int_rn(roundf(t)) + 128;       // roundf: half away from zero
                qi = max(0, min(255, qi));
                packed |= uint32_t(qi) << (8 * k);
                const long long fx = __float2ll_rn(fminf(fmaxf(t, -1.0e6f), 1.0e6f) * DL_FX);
                if (qi > 0 && qi < 255) {
                    const long long edge = static_cast<long long>(2 * qi - 257) << 19;        // (qi - 128.5) * 2^20
                    atomicAdd(&my_sum[qi], (1ull << 40) | static_cast<unsigned long long>(fx - edge));
                } else {
                    atomicAdd(&s_edge_sum[qi ? 1 : 0], static_cast<unsigned long long>(fx));   // two's complement: wraps correctly for negatives
                    atomicAdd(&s_edge_cnt[qi ? 1 : 0], 1u);
                }
            }
        }
        if (full) *reinterpret_cast<uint32_t*>(q + i) = packed;     // q + chunk start is 4-byte aligned
        else for (int k = 0; k < 4 && i + k < hi; ++k) q[i + k] = uint8_t(packed >> (8 * k));
    }
    __syncthreads();
    if (threadIdx.x < 256) {
        const int b = threadIdx.x;
        long long ssum;
        unsigned scnt;
        if (b > 0 && b < 255) {
            unsigned long long packed = 0ull;
#pragma unroll
            for (int c = 0; c < COPIES; ++c) packed += s_sum[c][b];      // integer sums: order-free
            scnt = unsigned(packed >> 40);
            ssum = static_cast<long long>(packed & ((1ull << 40) - 1)) + static_cast<long long>(scnt) * (static_cast<long long>(2 * b - 257) << 19);
        } else {
            ssum = static_cast<long long>(s_edge_sum[b ? 1 : 0]);
            scnt = s_edge_cnt[b ? 1 : 0];
        }
        bin_sum[(long long)blockIdx.x * 256 + b] = ssum;
        bin_cnt[(long long)blockIdx.x * 256 + b] = scnt;
    }
}

// ---- pass 3: codebook[chunk][b] = mean of bin b, merged over the blocks of a chunk ----
__global__ void dl_finalize_kernel(const long long* __restrict__ bin_sum, const unsigned* __restrict__ bin_cnt,
                                   const float* __restrict__ sumsq_partial, long long n, long long first_chunk,
                                   float* __restrict__ lut) {
    const int cb = blockIdx.x, b = threadIdx.x;
    const long long chunk = first_chunk + cb;
    const long long lo = chunk * DL_CHUNK, hi = min(n, lo + (long long)DL_CHUNK);
    const float scale = dl_chunk_scale(sumsq_partial, cb, hi - lo);
    long long s = 0;
    unsigned c = 0;
    for (int k = 0; k < DL_BLOCKS_PER_CHUNK; ++k) {
        s += bin_sum[((long long)cb * DL_BLOCKS_PER_CHUNK + k) * 256 + b];
        c += bin_cnt[((long long)cb * DL_BLOCKS_PER_CHUNK + k) * 256 + b];
    }
    lut[chunk * 256 + b] = c ? float(double(s) / double(DL_FX) / double(c)) * scale : 0.f;
}

// ---- stage B: pull every rank's bytes for my slice, dequantise with that rank's codebook, sum ----
__global__ void __launch_bounds__(DL_THREADS) dl_reduce_pull_kernel(DlPeers p, long long n, long long first_chunk, long long n_chunks,
                                                                    float* __restrict__ reduced) {
    extern __shared__ float s_lut[];   // [world][256]
    const long long chunk = first_chunk + blockIdx.x / DL_BLOCKS_PER_CHUNK;
    if (chunk >= first_chunk + n_chunks) return;
    const int sub = blockIdx.x % DL_BLOCKS_PER_CHUNK;
    const long long lo = chunk * DL_CHUNK, hi = min(n, lo + (long long)DL_CHUNK);
    for (int i = threadIdx.x; i < p.world * 256; i += blockDim.x) s_lut[i] = p.lut[i >> 8][chunk * 256 + (i & 255)];
    __syncthreads();
    // 16 bytes per thread per peer when aligned
    const long long lo16 = (lo + 15) & ~15ll;
    for (long long i = lo + sub * DL_THREADS + threadIdx.x; i < min(lo16, hi); i += DL_BLOCKS_PER_CHUNK * DL_THREADS) {
        float acc = 0.f;
        for (int r = 0; r < p.world; ++r) acc += s_lut[r * 256 + p.q[r][i]];
        reduced[i - first_chunk * DL_CHUNK] = acc;
    }
    const long long nvec = (hi > lo16) ? (hi - lo16) / 16 : 0;
    for (long long v = sub * DL_THREADS + threadIdx.x; v < nvec; v += DL_BLOCKS_PER_CHUNK * DL_THREADS) {
        const long long i = lo16 + v * 16;
        float acc[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) acc[k] = 0.f;
        for (int r = 0; r < p.world; ++r) {
            const uint4 u = *reinterpret_cast<const uint4*>(p.q[r] + i);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int k = 0; k < 16; ++k) acc[k] += s_lut[r * 256 + ((w[k >> 2] >> (8 * (k & 3))) & 255)];
        }
        float* dst = reduced + (i - first_chunk * DL_CHUNK);
#pragma unroll
        for (int k = 0; k < 16; ++k) dst[k] = acc[k];
    }
    for (long long i = lo16 + nvec * 16 + sub * DL_THREADS + threadIdx.x; i < hi; i += DL_BLOCKS_PER_CHUNK * DL_THREADS) {
        float acc = 0.f;
        for (int r = 0; r < p.world; ++r) acc += s_lut[r * 256 + p.q[r][i]];
        reduced[i - first_chunk * DL_CHUNK] = acc;
    }
}

// ---- stage C: pull the owners' reduced bytes, dequantise, Nesterov outer step, refresh inner ----
__global__ void __launch_bounds__(DL_THREADS) dl_gather_nesterov_kernel(DlPeers p, long long n, long long total_chunks,
                                                                        float* __restrict__ outer, float* __restrict__ inner,
                                                                        float* __restrict__ mom, float lr, float mu, float* g_out) {
    __shared__ float s_lut[256];
    const long long chunk = blockIdx.x / DL_BLOCKS_PER_CHUNK;
    const int sub = blockIdx.x % DL_BLOCKS_PER_CHUNK;
    const long long per = (total_chunks + p.world - 1) / p.world;
    const int owner = int(chunk / per);
    const long long lo = chunk * DL_CHUNK, hi = min(n, lo + (long long)DL_CHUNK);
    if (threadIdx.x < 256) s_lut[threadIdx.x] = p.lut2[owner][chunk * 256 + threadIdx.x];
    __syncthreads();
    const uint8_t* src = p.q2[owner];
    const bool aligned = ((reinterpret_cast<uintptr_t>(outer) | reinterpret_cast<uintptr_t>(inner) | reinterpret_cast<uintptr_t>(mom) |
                           reinterpret_cast<uintptr_t>(g_out)) & 15) == 0 && (reinterpret_cast<uintptr_t>(src) & 3) == 0;
    for (long long i = lo + (sub * DL_THREADS + threadIdx.x) * 4ll; i < hi; i += DL_BLOCKS_PER_CHUNK * DL_THREADS * 4ll) {
        if (aligned && i + 3 < hi) {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(src + i);
            const float4 g = make_float4(s_lut[w & 255], s_lut[(w >> 8) & 255], s_lut[(w >> 16) & 255], s_lut[w >> 24]);
            if (g_out) *reinterpret_cast<float4*>(g_out + i) = g;
            if (outer) {
                float4 m = *reinterpret_cast<const float4*>(mom + i);
                float4 o = *reinterpret_cast<const float4*>(outer + i);
                m.x = mu * m.x + g.x; m.y = mu * m.y + g.y; m.z = mu * m.z + g.z; m.w = mu * m.w + g.w;
                o.x -= lr * (g.x + mu * m.x); o.y -= lr * (g.y + mu * m.y); o.z -= lr * (g.z + mu * m.z); o.w -= lr * (g.w + mu * m.w);
                *reinterpret_cast<float4*>(mom + i) = m;
                *reinterpret_cast<float4*>(outer + i) = o;
                *reinterpret_cast<float4*>(inner + i) = o;
            }
        } else {
            for (long long j = i; j < min(hi, i + 4); ++j) {
                const float g = s_lut[src[j]];
                if (g_out) g_out[j] = g;
                if (outer) {
                    const float m = mu * mom[j] + g;
                    mom[j] = m;
                    const float o = outer[j] - lr * (g + mu * m);
                    outer[j] = o;
                    inner[j] = o;
                }
            }
        }
    }
}

}  // namespace pb

using namespace pb;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int pb_dl_chunk() { return DL_CHUNK; }
extern "C" int pb_dl_blocks_per_chunk() { return DL_BLOCKS_PER_CHUNK; }

static DlPeers make_dl_peers(int world, int rank, void* const* q, void* const* lut, void* const* q2, void* const* lut2) {
    DlPeers p{};
    p.world = world; p.rank = rank;
    for (int r = 0; r < world; ++r) {
        p.q[r] = (const uint8_t*)q[r]; p.lut[r] = (const float*)lut[r];
        p.q2[r] = (const uint8_t*)q2[r]; p.lut2[r] = (const float*)lut2[r];
    }
    return p;
}

// Stage A. scratch: partial [chunks*BPC] floats, bin_sum [chunks*BPC*256] int64, bin_cnt same (uint32).
// outer/inner: fp32 [n] device buffers. Writes q [n] and lut [chunks*256] (this rank's symmetric buffers).
extern "C" int pb_dl_stage_a(const float* outer, const float* inner, long long n, int world, int fake, void* q, float* lut,
                             float* partial, long long* bin_sum, unsigned* bin_cnt, void* stream) {
    const long long chunks = (n + DL_CHUNK - 1) / DL_CHUNK;
    const unsigned grid = unsigned(chunks * DL_BLOCKS_PER_CHUNK);
    const float inv_w = 1.f / float(world);
    dl_sumsq_kernel<0><<<grid, DL_THREADS, 0, ST(stream)>>>(outer, inner, inv_w, fake, n, 0, partial);
    dl_quantize_kernel<0><<<grid, DL_THREADS, 0, ST(stream)>>>(outer, inner, inv_w, fake, n, 0, partial, (uint8_t*)q, bin_sum, bin_cnt);
    dl_finalize_kernel<<<unsigned(chunks), 256, 0, ST(stream)>>>(bin_sum, bin_cnt, partial, n, 0, lut);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

// Stage B: reduce my slice of chunks by pulling from all ranks, then quantise it once into q2 / lut2.
// reduced: fp32 scratch of >= slice elements.
extern "C" int pb_dl_stage_b(void* const* q, void* const* lut, void* const* q2, void* const* lut2, int world, int rank, long long n,
                             float* reduced, float* partial, long long* bin_sum, unsigned* bin_cnt, void* stream) {
    if (world > DL_MAX_RANKS) return -1;
    const long long chunks = (n + DL_CHUNK - 1) / DL_CHUNK;
    const long long per = (chunks + world - 1) / world;
    const long long first = min(chunks, per * rank), mine = min(chunks, first + per) - first;
    if (mine <= 0) return 0;
    DlPeers p = make_dl_peers(world, rank, q, lut, q2, lut2);
    const unsigned grid = unsigned(mine * DL_BLOCKS_PER_CHUNK);
    dl_reduce_pull_kernel<<<grid, DL_THREADS, world * 256 * sizeof(float), ST(stream)>>>(p, n, first, mine, reduced);
    dl_sumsq_kernel<1><<<grid, DL_THREADS, 0, ST(stream)>>>(reduced, nullptr, 1.f, 0, n, first, partial);
    dl_quantize_kernel<1><<<grid, DL_THREADS, 0, ST(stream)>>>(reduced, nullptr, 1.f, 0, n, first, partial, (uint8_t*)q2[rank], bin_sum,
                                                             bin_cnt);
    dl_finalize_kernel<<<unsigned(mine), 256, 0, ST(stream)>>>(bin_sum, bin_cnt, partial, n, first, (float*)lut2[rank]);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

// Stage C: gather + Nesterov. outer/inner/mom may be null with g_out set (plain all-reduce result).
extern "C" int pb_dl_stage_c(void* const* q, void* const* lut, void* const* q2, void* const* lut2, int world, int rank, long long n,
                             float* outer, float* inner, float* mom, float lr, float mu, float* g_out, void* stream) {
    if (world > DL_MAX_RANKS) return -1;
    const long long chunks = (n + DL_CHUNK - 1) / DL_CHUNK;
    DlPeers p = make_dl_peers(world, rank, q, lut, q2, lut2);
    dl_gather_nesterov_kernel<<<unsigned(chunks * DL_BLOCKS_PER_CHUNK), DL_THREADS, 0, ST(stream)>>>(p, n, chunks, outer, inner, mom, lr,
                                                                                                     mu, g_out);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}
