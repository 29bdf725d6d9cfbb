// DiLoCo outer step on the GPU: pseudo-gradient, uint8 quantisation, all-reduce over NVLink peer
// memory with fp32 accumulation, and the Nesterov outer update — three kernels that read and write
// the peers' symmetric buffers directly and order themselves through per-peer epoch flags.
//
// Reference path being replaced: per-parameter device->host copies, CPU subtraction, the C++ gloo
// ring with a CPU quantiser, torch CPU SGD, host->device copies (src/zeroband/diloco.py:77-144,
// 203-215; C/csrc/collectives.cpp:76-230; C/csrc/compression.cpp:9-125).
//
// Group = the ranks that hold the same parameter shard in the workers; the ACTIVE members of one call are
// a bit mask (a worker that left is simply not in it, a worker that just joined contributes zeros once).
// NVSwitch gives uniform all-to-all bandwidth, so instead of a ring the exchange is direct:
//   stage A (local)   d = (outer - inner) * s   [0 for a "fake" joiner]; per 16 Ki-element chunk, one CTA of 512 threads,
//                     the chunk held in registers from the first read to the last write:
//                     sigma from the un-centred L2 norm, scale = 6 sigma / 256,
//                     q = clamp(round(d / scale) + 128), codebook[b] = mean of members of bin b
//                     -> q (uint8) and codebooks land in this rank's symmetric buffer; one HBM read of the
//                     inputs, one write of the bytes
//   stage B (pull)    the m active ranks split the chunks; the owner of a chunk sums codebook_p[q_p[i]] over
//                     all active ranks p in fp32 (fixed rank order) in registers and quantises the sum ONCE into
//                     its second symmetric buffer — the reduced fp32 values never go to memory
//   stage C (pull)    every rank reads every owner's reduced bytes + codebook, dequantises to g and
//                     applies  m = mu*m + g ; outer -= lr*(g + mu*m) ; inner = outer   (or just writes g)
// Values are quantised twice in total (reference: W-1 times plus a re-quantisation per all-gather
// hop), and all ranks decode the same bytes, so they end bit-identical. Quantiser semantics follow
// the reference (round half away from zero, empty bin -> 0, codebook = mean of the bin's members).
// Bin sums are integers (fixed point), so codebooks are bit-reproducible run to run.
// Ordering: the last CTA of a stage publishes "stage done, epoch e" to every active peer's flag pad
// (st.release.sys); the next stage's CTAs wait for the flags they depend on with a bounded spin that reports
// PB_ERR_TIMEOUT_PEER through the status word and skips the work instead of hanging. Membership only ever
// changes between calls, on the host. There is no multicast TMA and no library collective here.
#include "common.cuh"

namespace pb {

constexpr int DL_MAX_RANKS = 16;
constexpr int DL_CHUNK = 16384;           // elements per quantisation chunk = one CTA's register-resident tile
constexpr int DL_THREADS = 512;           // two CTAs per SM: one loads or waits at a barrier while the other computes
constexpr int DL_PER_THREAD = DL_CHUNK / DL_THREADS;   // 32
constexpr int DL_TABLE = 256 * 32;        // words of the CTA's shared table: 256 entries x one copy per lane (32 KB)
// One 32-bit shared-memory atomic per element: an inner bin holds (count << 20) | sum of the 9-bit fixed-point
// offsets of its members from the bin's lower edge. The histogram has one copy per lane (word bin * 32 + lane), so the 32
// atomics of a warp instruction always go to 32 different banks and never to the same word, whatever the values are.
// A copy sees the 512 elements that the threads with that lane number hold, so the count fits 10 bits and the sum
// (<= 512 * 512) fits 20; integer sums do not depend on the order of arrival, so codebooks are bit-reproducible.
// The offset resolution (1/512 of a bin width) puts the codebook entries within 1/1024 of a bin width of the exact mean.
constexpr int DL_FX_BITS = 9;
constexpr int DL_CNT_SHIFT = 20;
constexpr int DL_EDGE_FX_BITS = 14;       // the two clamping bins keep exact 64-bit sums at this resolution
constexpr int DL_FLAG_STRIDE = 16;        // ints per flag slot in a rank's pad (one per peer)

struct DlPeers {
    int world, rank;
    unsigned mask;                        // active ranks of this call
    uint8_t* q[DL_MAX_RANKS];             // stage A bytes of every rank   [n]
    float* lut[DL_MAX_RANKS];             // stage A codebooks             [chunks][256]
    uint8_t* q2[DL_MAX_RANKS];            // stage B bytes (owner slices)  [n]
    float* lut2[DL_MAX_RANKS];            // stage B codebooks             [chunks][256]
    int* flags[DL_MAX_RANKS];             // flag pads: int [slots][DL_FLAG_STRIDE]
    int slot_a, slot_b, slot_c;           // flag slots: stage A / B / C of an epoch are done on the writing rank
};

__device__ __forceinline__ void dl_st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int dl_ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Called by every thread of every CTA at the end of a stage: the last CTA to get here tells every active peer
// (and this rank itself) that the stage of `epoch` is complete on this rank, and re-arms the counter.
__device__ __forceinline__ void dl_publish_done(const DlPeers& p, int slot, int epoch, unsigned* counter) {
    __shared__ unsigned s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(counter, 1u) == gridDim.x - 1) ? 1u : 0u;
    __syncthreads();
    if (s_last && threadIdx.x == 0) {     // the thread that saw the last arrival publishes (release is cumulative over what it observed)
        *counter = 0u;
        __threadfence_system();
        for (int r = 0; r < p.world; ++r)
            if ((p.mask >> r) & 1u) dl_st_release_sys(p.flags[r] + slot * DL_FLAG_STRIDE + p.rank, epoch);
    }
}

// Wait (bounded) until every active peer has published `epoch` (or later) in `slot` of this rank's pad.
// Returns false for the whole CTA when a peer did not show up in time.
__device__ __forceinline__ bool dl_wait_peers(const DlPeers& p, int slot, int epoch, int* status, unsigned long long budget_ns) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (epoch > 0 && threadIdx.x < p.world && ((p.mask >> threadIdx.x) & 1u)) {
        const int* mine = p.flags[p.rank] + slot * DL_FLAG_STRIDE + threadIdx.x;
        const uint64_t t0 = globaltimer_ns();
        while (dl_ld_acquire_sys(mine) < epoch) {
            if (globaltimer_ns() - t0 > budget_ns) {
                if (status) atomicCAS(status, 0, PB_ERR_TIMEOUT_PEER | (int(threadIdx.x) << 8));
                s_ok = 0;
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    const bool ok = s_ok != 0;
    __syncthreads();       // everyone has read the verdict before a later call re-arms the shared word
    return ok;
}

__device__ __forceinline__ float dl_block_sum(float v) {
    __shared__ float red[DL_THREADS / 32];
    __shared__ float total;
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < DL_THREADS / 32; ++i) t += red[i];      // fixed order
        total = t;
    }
    __syncthreads();
    return total;
}

// Quantise the CTA's register-resident chunk and write bytes + codebook. Thread t holds 32 / G groups of G
// consecutive elements: element (k*512 + t)*G + j sits in v[G*k + j] (G = 4 after the fp32 loads of stage A, G = 16 after
// the byte loads of stage B). `cnt` = valid elements of the chunk.
// Rounding without the conversion unit: adding 1.5 * 2^23 to |t| < 2^22 leaves round-to-nearest-even(t) in the low
// mantissa bits of the sum.
constexpr float DL_MAGIC = 12582912.f;
constexpr int DL_MAGIC_BITS = 0x4B400000;

template <int G, bool FULL>
__device__ __forceinline__ void dl_quantize_body(const float (&v)[DL_PER_THREAD], int cnt, uint8_t* __restrict__ q_chunk,
                                                 bool q_aligned, unsigned* my_bin, long long (&e_sum)[2], unsigned (&e_cnt)[2],
                                                 float inv_scale) {
#pragma unroll
    for (int k = 0; k < DL_PER_THREAD / G; ++k) {
        const int e0 = (k * DL_THREADS + int(threadIdx.x)) * G;
        uint32_t w[G / 4];
#pragma unroll
        for (int j = 0; j < G / 4; ++j) w[j] = 0u;
#pragma unroll
        for (int j = 0; j < G; ++j) {
            int qi = 128;                                                 // elements past the end pack as the zero bin
            if (FULL || e0 + j < cnt) {
                const float t = v[G * k + j] * inv_scale;
                const float m = t + DL_MAGIC;
                qi = __float_as_int(m) - (DL_MAGIC_BITS - 128);           // nearest bin (a tie, one value in ~10^7, goes to the even one);
                                                                          // far outside the magic range the sign and a large magnitude survive
                const float d = t - (m - DL_MAGIC);                       // in [-0.5, 0.5] inside the range
                qi = max(0, min(255, qi));
                if (unsigned(qi - 1) < 254u) {
                    // (count 1 << 20) | offset from the bin's lower edge as 9-bit fixed point: one fused multiply-add and one add
                    const unsigned val = unsigned(__float_as_int(d * float(1 << DL_FX_BITS) + (DL_MAGIC + float(1 << (DL_FX_BITS - 1)))) -
                                                  (DL_MAGIC_BITS - (1 << DL_CNT_SHIFT)));
                    atomicAdd(&my_bin[qi << 5], val);
                } else {
                    // the two clamping bins take values from an unbounded range: exact 64-bit sums of their own, kept
                    // per thread (about one element in 400 lands here) and combined once per chunk
                    const long long fx = __float2ll_rn(fminf(fmaxf(t, -1.0e6f), 1.0e6f) * float(1 << DL_EDGE_FX_BITS));
                    if (qi) { e_sum[1] += fx; ++e_cnt[1]; }
                    else { e_sum[0] += fx; ++e_cnt[0]; }
                }
            }
            w[j >> 2] = __funnelshift_r(w[j >> 2], uint32_t(qi), 8);      // bytes enter at the top: after four, element j sits in byte j & 3
        }
        if (q_aligned && (FULL || e0 + G - 1 < cnt)) {
            if (G == 4) *reinterpret_cast<uint32_t*>(q_chunk + e0) = w[0];
            else *reinterpret_cast<uint4*>(q_chunk + e0) = make_uint4(w[0], w[1 % (G / 4)], w[2 % (G / 4)], w[3 % (G / 4)]);
        } else {
            for (int j = 0; j < G && e0 + j < cnt; ++j) q_chunk[e0 + j] = uint8_t(w[j >> 2] >> (8 * (j & 3)));
        }
    }
}

template <int G>
__device__ __forceinline__ void dl_quantize_chunk(float (&v)[DL_PER_THREAD], long long cnt, uint8_t* __restrict__ q_chunk,
                                                  float* __restrict__ lut_chunk, bool q_aligned, unsigned* s_bin) {
    __shared__ unsigned long long s_edge_sum[2];
    __shared__ unsigned s_edge_cnt[2];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < DL_PER_THREAD; ++i) ss += v[i] * v[i];
    __syncthreads();                                         // the table's previous use (look-ups, last chunk's codebook) is over
    for (int i = threadIdx.x; i < DL_TABLE; i += DL_THREADS) s_bin[i] = 0u;
    if (threadIdx.x < 2) { s_edge_sum[threadIdx.x] = 0ull; s_edge_cnt[threadIdx.x] = 0u; }
    ss = dl_block_sum(ss);                                   // also orders the zeroing above before the atomics below
    const float sigma = sqrtf(ss / float(cnt > 1 ? cnt - 1 : 1));
    float scale = 6.f * sigma / 256.f;
    if (!(scale > 0.f) || isinf(scale)) scale = 1.f;         // all-zero chunk (e.g. a fake pseudo-gradient)
    const float inv_scale = 1.f / scale;
    unsigned* my_bin = s_bin + (threadIdx.x & 31);
    long long e_sum[2] = {0ll, 0ll};
    unsigned e_cnt[2] = {0u, 0u};
    if (cnt == DL_CHUNK) dl_quantize_body<G, true>(v, DL_CHUNK, q_chunk, q_aligned, my_bin, e_sum, e_cnt, inv_scale);
    else dl_quantize_body<G, false>(v, int(cnt), q_chunk, q_aligned, my_bin, e_sum, e_cnt, inv_scale);
#pragma unroll
    for (int b = 0; b < 2; ++b) {                            // one shared atomic per warp and clamping bin, and only if it has members
        unsigned c = e_cnt[b];
        long long sm = e_sum[b];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            c += __shfl_xor_sync(0xffffffffu, c, o);
            sm += __shfl_xor_sync(0xffffffffu, sm, o);
        }
        if ((threadIdx.x & 31) == 0 && c) {
            atomicAdd(&s_edge_sum[b], static_cast<unsigned long long>(sm));
            atomicAdd(&s_edge_cnt[b], c);
        }
    }
    __syncthreads();
    if (threadIdx.x < 256) {
        const int b = threadIdx.x;
        float mean = 0.f;
        if (b > 0 && b < 255) {
            unsigned long long sum = 0;
            unsigned c = 0;
#pragma unroll
            for (int l = 0; l < 32; ++l) {
                const unsigned x = s_bin[(b << 5) + ((l + b) & 31)];      // rotated: the 32 bins of a warp read 32 different banks
                c += x >> DL_CNT_SHIFT;
                sum += x & ((1u << DL_CNT_SHIFT) - 1u);
            }
            if (c) mean = (float(b) - 128.5f + float(double(sum) / double(1 << DL_FX_BITS) / double(c))) * scale;
        } else {
            const unsigned c = s_edge_cnt[b ? 1 : 0];
            if (c) mean = float(double(static_cast<long long>(s_edge_sum[b ? 1 : 0])) / double(1 << DL_EDGE_FX_BITS) / double(c)) * scale;
        }
        lut_chunk[b] = mean;
    }
    __syncthreads();       // the shared table is reused by the CTA's next chunk
}

// ---- stage A: value -> registers -> bytes + codebook ----
// value = (a - b) * s, or a * s when b is null, or 0 if fake.
__global__ void __launch_bounds__(DL_THREADS, 2) dl_stage_a_kernel(DlPeers p, const float* __restrict__ a, const float* __restrict__ b, float s,
                                                                int fake, long long n, int epoch, unsigned* counter, int signal) {
    const long long chunks = (n + DL_CHUNK - 1) / DL_CHUNK;
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
    uint8_t* q = p.q[p.rank];
    float* lut = p.lut[p.rank];
    const bool q_aligned = (reinterpret_cast<uintptr_t>(q) & 3) == 0;
    __shared__ unsigned s_tab[DL_TABLE];
    for (long long chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
        const long long lo = chunk * DL_CHUNK;
        const long long cnt = min((long long)DL_CHUNK, n - lo);
        float v[DL_PER_THREAD];
#pragma unroll
        for (int k = 0; k < DL_PER_THREAD / 4; ++k) {
            const long long e0 = (long long)(k * DL_THREADS + threadIdx.x) * 4;
            float x[4] = {0.f, 0.f, 0.f, 0.f};
            if (!fake) {
                if (aligned && e0 + 3 < cnt) {
                    const float4 t = __ldcs(reinterpret_cast<const float4*>(a + lo + e0));
                    x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
                    if (b) {
                        const float4 u = __ldcs(reinterpret_cast<const float4*>(b + lo + e0));
                        x[0] -= u.x; x[1] -= u.y; x[2] -= u.z; x[3] -= u.w;
                    }
                } else {
                    for (int j = 0; j < 4 && e0 + j < cnt; ++j) x[j] = b ? a[lo + e0 + j] - b[lo + e0 + j] : a[lo + e0 + j];
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) v[4 * k + j] = x[j] * s;
        }
        dl_quantize_chunk<4>(v, cnt, q + lo, lut + chunk * 256, q_aligned, s_tab);
    }
    if (signal) dl_publish_done(p, p.slot_a, epoch, counter);
}

// rank that owns `chunk` when the `m` active ranks of `mask` split `chunks` chunks into contiguous runs of `per`
__device__ __forceinline__ int dl_owner(unsigned mask, long long chunk, long long per) {
    int idx = int(chunk / per);
    int r = 0;
    for (;; ++r) {
        if ((mask >> r) & 1u) {
            if (idx == 0) break;
            --idx;
        }
    }
    return r;
}

// ---- stage B: pull every active rank's bytes for my chunks, dequantise with that rank's codebook, sum, re-quantise ----
__global__ void __launch_bounds__(DL_THREADS, 2) dl_stage_b_kernel(DlPeers p, long long n, int epoch, int prev_epoch, unsigned* counter,
                                                                int* status, unsigned long long budget_ns) {
    __shared__ unsigned s_tab[DL_TABLE];   // histogram of the re-quantisation
    extern __shared__ float s_lut[];       // [world][256]: every active rank's codebook of the current chunk
    const long long chunks = (n + DL_CHUNK - 1) / DL_CHUNK;
    const int m = __popc(p.mask);
    const long long per = (chunks + m - 1) / m;
    const int my_idx = __popc(p.mask & ((1u << p.rank) - 1u));
    const long long first = min(chunks, per * my_idx), last = min(chunks, first + per);
    // my stage-A output is read by peers during their stage B, and my q2 / lut2 (written below) are read by peers during
    // stage C of the previous call: wait for "A done, this epoch" and "C done, previous epoch" from every active rank
    bool ok = dl_wait_peers(p, p.slot_a, epoch, status, budget_ns);
    ok = dl_wait_peers(p, p.slot_c, prev_epoch, status, budget_ns) && ok;
    uint8_t* q2 = p.q2[p.rank];
    float* lut2 = p.lut2[p.rank];
    const bool vec_ok = (reinterpret_cast<uintptr_t>(p.q[0]) & 15) == 0;    // symmetric buffers share their alignment
    for (long long chunk = first + blockIdx.x; ok && chunk < last; chunk += gridDim.x) {
        const long long lo = chunk * DL_CHUNK;
        const long long cnt = min((long long)DL_CHUNK, n - lo);
        __syncthreads();                   // the previous chunk's look-ups are over
        for (int i = threadIdx.x; i < p.world * 256; i += DL_THREADS) {
            const int r = i >> 8;
            s_lut[i] = ((p.mask >> r) & 1u) ? p.lut[r][chunk * 256 + (i & 255)] : 0.f;
        }
        __syncthreads();
        // thread t owns the 16-element groups g = k*512 + t, k = 0..1: one 16-byte load per peer and group
        float acc[DL_PER_THREAD];
#pragma unroll
        for (int i = 0; i < DL_PER_THREAD; ++i) acc[i] = 0.f;
        for (int r = 0; r < p.world; ++r) {
            if (!((p.mask >> r) & 1u)) continue;
            const uint8_t* src = p.q[r] + lo;
            const float* L = s_lut + r * 256;
#pragma unroll
            for (int k = 0; k < DL_PER_THREAD / 16; ++k) {
                const long long e0 = (long long)(k * DL_THREADS + threadIdx.x) * 16;
                if (vec_ok && e0 + 15 < cnt) {
                    const uint4 u = *reinterpret_cast<const uint4*>(src + e0);
                    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[16 * k + j] += L[(w[j >> 2] >> (8 * (j & 3))) & 255];
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (e0 + j < cnt) acc[16 * k + j] += L[src[e0 + j]];
                }
            }
        }
        // the fp32 sums stay in registers: quantised once more, bytes and codebook into this rank's second buffer
        dl_quantize_chunk<16>(acc, cnt, q2 + lo, lut2 + chunk * 256, (reinterpret_cast<uintptr_t>(q2) & 15) == 0, s_tab);
    }
    dl_publish_done(p, p.slot_b, epoch, counter);
}

// ---- stage C: pull the owners' reduced bytes, dequantise, Nesterov outer step, refresh inner (or write g) ----
__global__ void __launch_bounds__(DL_THREADS, 2) dl_stage_c_kernel(DlPeers p, long long n, float* __restrict__ outer, float* __restrict__ inner,
                                                                float* __restrict__ mom, float lr, float mu, float* __restrict__ g_out,
                                                                int epoch, unsigned* counter, int* status, unsigned long long budget_ns) {
    __shared__ float s_lut[256];           // the owner's codebook of the current chunk
    const long long chunks = (n + DL_CHUNK - 1) / DL_CHUNK;
    const int m = __popc(p.mask);
    const long long per = (chunks + m - 1) / m;
    const bool ok = dl_wait_peers(p, p.slot_b, epoch, status, budget_ns);
    const bool aligned = ((reinterpret_cast<uintptr_t>(outer) | reinterpret_cast<uintptr_t>(inner) | reinterpret_cast<uintptr_t>(mom) |
                           reinterpret_cast<uintptr_t>(g_out)) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.q2[0]) & 15) == 0;
    for (long long chunk = blockIdx.x; ok && chunk < chunks; chunk += gridDim.x) {
        const int owner = dl_owner(p.mask, chunk, per);
        const long long lo = chunk * DL_CHUNK;
        const long long cnt = min((long long)DL_CHUNK, n - lo);
        __syncthreads();
        if (threadIdx.x < 256) s_lut[threadIdx.x] = p.lut2[owner][chunk * 256 + threadIdx.x];
        __syncthreads();
        const uint8_t* src = p.q2[owner] + lo;
#pragma unroll 1
        for (int k = 0; k < DL_PER_THREAD / 16; ++k) {
            const long long e0 = (long long)(k * DL_THREADS + threadIdx.x) * 16;
            if (aligned && e0 + 15 < cnt) {
                const uint4 u = *reinterpret_cast<const uint4*>(src + e0);
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const long long i = lo + e0 + 4 * h;
                    const float4 g = make_float4(s_lut[w[h] & 255], s_lut[(w[h] >> 8) & 255], s_lut[(w[h] >> 16) & 255], s_lut[w[h] >> 24]);
                    if (g_out) __stcs(reinterpret_cast<float4*>(g_out + i), g);
                    if (outer) {
                        float4 mm = __ldcs(reinterpret_cast<const float4*>(mom + i));
                        float4 o = __ldcs(reinterpret_cast<const float4*>(outer + i));
                        mm.x = mu * mm.x + g.x; mm.y = mu * mm.y + g.y; mm.z = mu * mm.z + g.z; mm.w = mu * mm.w + g.w;
                        o.x -= lr * (g.x + mu * mm.x); o.y -= lr * (g.y + mu * mm.y); o.z -= lr * (g.z + mu * mm.z); o.w -= lr * (g.w + mu * mm.w);
                        __stcs(reinterpret_cast<float4*>(mom + i), mm);
                        __stcs(reinterpret_cast<float4*>(outer + i), o);
                        __stcs(reinterpret_cast<float4*>(inner + i), o);
                    }
                }
            } else {
                for (int j = 0; j < 16 && e0 + j < cnt; ++j) {
                    const long long i = lo + e0 + j;
                    const float g = s_lut[src[e0 + j]];
                    if (g_out) g_out[i] = g;
                    if (outer) {
                        const float mm = mu * mom[i] + g;
                        mom[i] = mm;
                        const float o = outer[i] - lr * (g + mu * mm);
                        outer[i] = o;
                        inner[i] = o;
                    }
                }
            }
        }
    }
    dl_publish_done(p, p.slot_c, epoch, counter);
}

}  // namespace pb

using namespace pb;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int pb_dl_chunk() { return DL_CHUNK; }

static int dl_grid(long long chunks) {
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n_sm = 148;
    }
    const long long cap = 2LL * n_sm;          // two CTAs of 512 threads per SM (64 registers per thread), each looping over its chunks
    return int(chunks < cap ? (chunks > 0 ? chunks : 1) : cap);
}

// Local quantiser on its own: q [n] bytes and lut [chunks][256] of x (fp32, device). No peers, no flags.
extern "C" int pb_dl_quantize(const float* x, long long n, void* q, float* lut, void* stream) {
    DlPeers p{};
    p.world = 1; p.rank = 0; p.mask = 1u;
    p.q[0] = (uint8_t*)q; p.lut[0] = lut;
    const long long chunks = (n + DL_CHUNK - 1) / DL_CHUNK;
    dl_stage_a_kernel<<<dl_grid(chunks), DL_THREADS, 0, ST(stream)>>>(p, x, nullptr, 1.f, 0, n, 0, nullptr, 0);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

// The whole exchange: stage A, B and C back to back on `stream`.
//   value_i = (a_i - b_i) * scale (b may be null), 0 when fake
//   q / lut / q2 / lut2 / flags: per-rank pointer tables of the symmetric buffers and flag pads
//   mask: active ranks of this call (bit r); this rank must be in it
//   epoch: strictly increasing per group; prev_epoch: epoch of the previous call of this group (0 after a host-side
//   rendezvous, e.g. at start-up or when the membership changed)
//   slot_base: first of three consecutive flag slots reserved for this group
//   counters: three zero-initialised device words (re-armed by the kernels)
//   outer / inner / mom (Nesterov outer step in place, inner := outer) and / or g_out (the averaged value), fp32 [n]
//   budget_ns: how long a wait for a peer may spin before the call gives up with PB_ERR_TIMEOUT_PEER in *status
extern "C" int pb_dl_allreduce(void* const* q, void* const* lut, void* const* q2, void* const* lut2, void* const* flags, int world, int rank,
                               unsigned mask, int epoch, int prev_epoch, int slot_base, long long n, const float* a, const float* b,
                               float scale, int fake, float* outer, float* inner, float* mom, float lr, float mu, float* g_out,
                               unsigned* counters, int* status, long long budget_ns, void* stream) {
    if (world > DL_MAX_RANKS || world < 1 || !((mask >> rank) & 1u) || (mask >> world) != 0u || epoch <= 0) return -1;
    DlPeers p{};
    p.world = world; p.rank = rank; p.mask = mask;
    for (int r = 0; r < world; ++r) {
        p.q[r] = (uint8_t*)q[r]; p.lut[r] = (float*)lut[r]; p.q2[r] = (uint8_t*)q2[r]; p.lut2[r] = (float*)lut2[r];
        p.flags[r] = (int*)flags[r];
    }
    p.slot_a = slot_base; p.slot_b = slot_base + 1; p.slot_c = slot_base + 2;
    const long long chunks = (n + DL_CHUNK - 1) / DL_CHUNK;
    const int m = __builtin_popcount(mask);
    const long long per = (chunks + m - 1) / m;
    const unsigned long long budget = budget_ns > 0 ? (unsigned long long)budget_ns : PB_WAIT_BUDGET_NS;
    dl_stage_a_kernel<<<dl_grid(chunks), DL_THREADS, 0, ST(stream)>>>(p, a, b, scale, fake, n, epoch, counters, 1);
    dl_stage_b_kernel<<<dl_grid(per), DL_THREADS, world * 256 * sizeof(float), ST(stream)>>>(p, n, epoch, prev_epoch, counters + 1, status,
                                                                                          budget);
    dl_stage_c_kernel<<<dl_grid(chunks), DL_THREADS, 0, ST(stream)>>>(p, n, outer, inner, mom, lr, mu, g_out, epoch, counters + 2, status,
                                                                     budget);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}
