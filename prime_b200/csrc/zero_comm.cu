// ZeRO-3 collectives fused with their consumers, over NVLink peer memory (symmetric buffers).
//
// Each rank holds the full bf16/fp32 gradient buffer it just produced in symmetric memory and a
// table `peers[r]` of every rank's copy of that buffer. The reference does this with FSDP2 +
// NCCL reduce-scatter / all-gather plus separate foreach kernels (src/zeroband/train.py:150-168,
// 365-372); here the collective is executed by the kernel that also does the math:
//
//   pb_zero_reduce_grads : reduce-scatter by PULL. For every segment this rank owns, load the
//                          slice from all W ranks with plain P2P ld.global (every thread has the
//                          loads of all W peers in flight before its first add, so all links are
//                          busy at once), sum in fp32 in fixed rank order (bit-identical on every
//                          run), scale, write the fp32 shard and accumulate the sum of squares
//                          needed for global-norm clipping.
//   pb_zero_adamw_gather : sharded AdamW fused with the all-gather by PUSH. Each updated value is
//                          converted to bf16 and stored straight into every rank's parameter
//                          buffer with P2P st.global, so no gathered copy is ever staged.
//   pb_peer_barrier      : one-CTA epoch barrier on per-peer flags (st.release.sys / ld.acquire.sys)
//                          with a bounded spin that reports PB_ERR_TIMEOUT_PEER instead of hanging.
//   pb_allreduce_scalars : all-reduce of a few fp32 scalars through the flag pads, summed in rank
//                          order so every rank gets the same bits.
// No TMA multicast and no library collective is involved anywhere in this file.
#include "common.cuh"

namespace pb {

constexpr int MAX_SEGS = 128;   // one launch can cover every parameter of a model with up to ~14 blocks; tables are kernel arguments
constexpr int MAX_RANKS = 16;

struct SegTable {
    int n;
    long long full_off[MAX_SEGS];
    long long shard_off[MAX_SEGS];
    long long numel[MAX_SEGS];
    // CTAs [cta_begin[s], cta_begin[s + 1]) work on segment s, in proportion to its size, so that all segments of
    // a launch stream at once (a grid-stride pass of the whole grid over one small segment leaves most of it idle)
    int cta_begin[MAX_SEGS + 1];
};
// this CTA's segment and its position among the CTAs of that segment
__device__ __forceinline__ void my_segment(const SegTable& segs, int& s, long long& b, long long& nb) {
    s = 0;
    while (s + 1 < segs.n && int(blockIdx.x) >= segs.cta_begin[s + 1]) ++s;
    b = blockIdx.x - segs.cta_begin[s];
    nb = segs.cta_begin[s + 1] - segs.cta_begin[s];
}
struct PeerTable {
    int world, rank;
    void* ptr[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// pads[r] points at rank r's flag pad: int[slots][MAX_RANKS]. Thread t signals peer t and waits
// for peer t's signal in its own pad. Epochs only grow, so no reset race exists.
__global__ void peer_barrier_kernel(PeerTable pads, int slot, int epoch, int* status, unsigned long long budget_ns) {
    const int t = threadIdx.x;
    if (t >= pads.world) return;
    __threadfence_system();
    int* remote = reinterpret_cast<int*>(pads.ptr[t]) + slot * MAX_RANKS + pads.rank;
    st_release_sys(remote, epoch);
    const int* mine = reinterpret_cast<const int*>(pads.ptr[pads.rank]) + slot * MAX_RANKS + t;
    const uint64_t t0 = globaltimer_ns();
    while (ld_acquire_sys(mine) < epoch) {
        if (globaltimer_ns() - t0 > budget_ns) {
            if (status) atomicCAS(status, 0, PB_ERR_TIMEOUT_PEER | (t << 8));
            return;
        }
        __nanosleep(200);
    }
}

// vals[pads.rank][slot][0..n) of every rank -> summed into out[0..n), identical order everywhere.
// data pads: float[slots][2 (epoch parity)][MAX_RANKS][8]; the parity double-buffer lets a fast rank start
// the next reduction while a slow one still sums the previous values
__global__ void allreduce_scalars_kernel(PeerTable flag_pads, PeerTable data_pads, int slot, int epoch,
                                         const float* __restrict__ in, float* __restrict__ out, int n, int* status,
                                         unsigned long long budget_ns) {
    const int t = threadIdx.x;
    if (t < flag_pads.world) {
        float* remote = reinterpret_cast<float*>(data_pads.ptr[t]) + ((slot * 2 + (epoch & 1)) * MAX_RANKS + flag_pads.rank) * 8;
        for (int i = 0; i < n; ++i) remote[i] = in[i];
        __threadfence_system();
        st_release_sys(reinterpret_cast<int*>(flag_pads.ptr[t]) + slot * MAX_RANKS + flag_pads.rank, epoch);
        const int* mine = reinterpret_cast<const int*>(flag_pads.ptr[flag_pads.rank]) + slot * MAX_RANKS + t;
        const uint64_t t0 = globaltimer_ns();
        bool ok = true;
        while (ld_acquire_sys(mine) < epoch) {
            if (globaltimer_ns() - t0 > budget_ns) {
                if (status) atomicCAS(status, 0, PB_ERR_TIMEOUT_PEER | (t << 8));
                ok = false;
                break;
            }
            __nanosleep(200);
        }
        (void)ok;
    }
    __syncthreads();
    if (t < n) {
        const volatile float* mine = reinterpret_cast<const volatile float*>(data_pads.ptr[flag_pads.rank]) + (slot * 2 + (epoch & 1)) * MAX_RANKS * 8;
        float s = 0.f;
        for (int r = 0; r < flag_pads.world; ++r) s += mine[r * 8 + t];
        out[t] = s;
    }
}

template <typename G>
__device__ __forceinline__ float ld_grad(const G* p) { return float(*p); }

// Sum of `nvec` 8-element bf16 vectors over the W ranks (rank order), scaled, written as fp32; returns this
// thread's sum of squares. UNR vectors per thread and step with every peer load issued before the first add:
// enough bytes in flight for HBM (one rank) and for NVLink (several ranks) alike.
template <int WMAX, int UNR>
__device__ __forceinline__ float reduce_vectors(const PeerTable& peers, int W, long long fo, long long nvec, float scale,
                                                float* __restrict__ dst, long long b, long long nb) {
    float ss = 0.f;
    const long long stride = nb * blockDim.x;
    for (long long i0 = b * blockDim.x + threadIdx.x; i0 < nvec; i0 += UNR * stride) {
        uint4 v[UNR][WMAX];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const long long i = i0 + u * stride;
#pragma unroll
            for (int r = 0; r < WMAX; ++r)
                if (r < W && i < nvec) v[u][r] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(peers.ptr[r]) + fo) + i);
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const long long i = i0 + u * stride;
            if (i < nvec) {
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
                for (int r = 0; r < WMAX; ++r)
                    if (r < W) {
                        const float2 a = unpack_bf16x2(v[u][r].x), b = unpack_bf16x2(v[u][r].y), c = unpack_bf16x2(v[u][r].z), d = unpack_bf16x2(v[u][r].w);
                        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
                    }
#pragma unroll
                for (int k = 0; k < 8; ++k) { acc[k] *= scale; ss += acc[k] * acc[k]; }
                reinterpret_cast<float4*>(dst)[2 * i] = make_float4(acc[0], acc[1], acc[2], acc[3]);
                reinterpret_cast<float4*>(dst)[2 * i + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
            }
        }
    }
    return ss;
}

// Reduce-scatter by pull + cast/scale + sum of squares. grid-stride over the segment elements.
template <typename G>
__global__ void __launch_bounds__(256) zero_reduce_grads_kernel(PeerTable peers, SegTable segs, float* __restrict__ grad_shard,
                                                                float scale, float* __restrict__ sumsq_partial) {
    __shared__ float red[8];
    float ss = 0.f;
    const int W = peers.world;
    int s;
    long long b, nb;
    my_segment(segs, s, b, nb);
    if (nb > 0) {
        const long long n = segs.numel[s];
        const long long fo = segs.full_off[s];
        float* dst = grad_shard + segs.shard_off[s];
        // vector path: 8 elements per thread per step when everything is 16-byte aligned
        const bool vec_ok = (fo % 8 == 0) && (segs.shard_off[s] % 4 == 0) && sizeof(G) == 2;
        const long long nvec = vec_ok ? n / 8 : 0;
        if (W <= 4) ss += reduce_vectors<4, 4>(peers, W, fo, nvec, scale, dst, b, nb);
        else if (W <= 8) ss += reduce_vectors<8, 2>(peers, W, fo, nvec, scale, dst, b, nb);
        else ss += reduce_vectors<MAX_RANKS, 1>(peers, W, fo, nvec, scale, dst, b, nb);
        for (long long i = nvec * 8 + b * blockDim.x + threadIdx.x; i < n; i += nb * blockDim.x) {
            float acc = 0.f;
            for (int r = 0; r < W; ++r) acc += ld_grad(reinterpret_cast<const G*>(peers.ptr[r]) + fo + i);
            acc *= scale;
            ss += acc * acc;
            dst[i] = acc;
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < (blockDim.x >> 5); ++i) t += red[i];
        sumsq_partial[blockIdx.x] = t;
    }
}

// fixed-order sum of `n` partials -> out[0] (+)=
__global__ void reduce_partials_kernel(const float* __restrict__ partial, int n, float* __restrict__ out, int accumulate) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < n; ++i) t += partial[i];
        out[0] = accumulate ? out[0] + t : t;
    }
}

// Sharded AdamW + push all-gather. gnorm_sq: device scalar with the GLOBAL sum of squared grads.
__global__ void __launch_bounds__(256) zero_adamw_gather_kernel(PeerTable params, SegTable segs, float* __restrict__ master,
                                                                const float* __restrict__ grad_shard, float* __restrict__ m,
                                                                float* __restrict__ v, float lr, float beta1, float beta2, float eps,
                                                                float wd, float bc1, float bc2, const float* __restrict__ gnorm_sq,
                                                                float max_norm) {
    float clip = 1.f;
    if (gnorm_sq && max_norm > 0.f) {
        const float c = max_norm / (sqrtf(*gnorm_sq) + 1e-6f);
        clip = c < 1.f ? c : 1.f;
    }
    const int W = params.world;
    int s;
    long long b, nb;
    my_segment(segs, s, b, nb);
    if (nb > 0) {
        const long long n = segs.numel[s], fo = segs.full_off[s], so = segs.shard_off[s];
        const bool vec_ok = (fo % 8 == 0) && (so % 4 == 0);
        const long long nvec = vec_ok ? n / 8 : 0;
        // two 8-element vectors per thread and step: sixteen 16-byte streaming loads are issued before the first use
        const long long stride = nb * blockDim.x;
        for (long long i0 = b * blockDim.x + threadIdx.x; i0 < nvec; i0 += 2 * stride) {
            float p[2][8], g[2][8], mm[2][8], vv[2][8];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const long long i = i0 + u * stride;
                if (i < nvec) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        *reinterpret_cast<float4*>(p[u] + 4 * h) = __ldcs(reinterpret_cast<const float4*>(master + so) + 2 * i + h);
                        *reinterpret_cast<float4*>(g[u] + 4 * h) = __ldcs(reinterpret_cast<const float4*>(grad_shard + so) + 2 * i + h);
                        *reinterpret_cast<float4*>(mm[u] + 4 * h) = __ldcs(reinterpret_cast<const float4*>(m + so) + 2 * i + h);
                        *reinterpret_cast<float4*>(vv[u] + 4 * h) = __ldcs(reinterpret_cast<const float4*>(v + so) + 2 * i + h);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const long long i = i0 + u * stride;
                if (i >= nvec) break;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float gi = g[u][k] * clip;
                    p[u][k] *= (1.f - lr * wd);
                    mm[u][k] = beta1 * mm[u][k] + (1.f - beta1) * gi;
                    vv[u][k] = beta2 * vv[u][k] + (1.f - beta2) * gi * gi;
                    p[u][k] -= (lr / bc1) * (mm[u][k] / (sqrtf(vv[u][k]) / bc2 + eps));
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    __stcs(reinterpret_cast<float4*>(master + so) + 2 * i + h, *reinterpret_cast<float4*>(p[u] + 4 * h));
                    __stcs(reinterpret_cast<float4*>(m + so) + 2 * i + h, *reinterpret_cast<float4*>(mm[u] + 4 * h));
                    __stcs(reinterpret_cast<float4*>(v + so) + 2 * i + h, *reinterpret_cast<float4*>(vv[u] + 4 * h));
                }
                uint4 o;
                o.x = pack_bf16x2(p[u][0], p[u][1]); o.y = pack_bf16x2(p[u][2], p[u][3]);
                o.z = pack_bf16x2(p[u][4], p[u][5]); o.w = pack_bf16x2(p[u][6], p[u][7]);
#pragma unroll
                for (int r = 0; r < MAX_RANKS; ++r)
                    if (r < W) {
                        const int dstr = (params.rank + r) % W;   // rotate so ranks push to different GPUs at once
                        reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.ptr[dstr]) + fo)[i] = o;
                    }
            }
        }
        for (long long i = nvec * 8 + b * blockDim.x + threadIdx.x; i < n; i += nb * blockDim.x) {
            const float gi = grad_shard[so + i] * clip;
            float pi = master[so + i] * (1.f - lr * wd);
            const float mi = beta1 * m[so + i] + (1.f - beta1) * gi;
            const float vi = beta2 * v[so + i] + (1.f - beta2) * gi * gi;
            pi -= (lr / bc1) * (mi / (sqrtf(vi) / bc2 + eps));
            master[so + i] = pi; m[so + i] = mi; v[so + i] = vi;
            const __nv_bfloat16 o = __float2bfloat16(pi);
            for (int r = 0; r < W; ++r) reinterpret_cast<__nv_bfloat16*>(params.ptr[(params.rank + r) % W])[fo + i] = o;
        }
    }
}

// master fp32 shard -> bf16 pushed into every rank's parameter buffer (initial broadcast / after a
// checkpoint load or a DiLoCo outer step rewrote the master shard)
__global__ void __launch_bounds__(256) zero_push_params_kernel(PeerTable params, SegTable segs, const float* __restrict__ master) {
    const int W = params.world;
    for (int s = 0; s < segs.n; ++s) {
        const long long n = segs.numel[s], fo = segs.full_off[s], so = segs.shard_off[s];
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
            const __nv_bfloat16 o = __float2bfloat16(master[so + i]);
            for (int r = 0; r < W; ++r) reinterpret_cast<__nv_bfloat16*>(params.ptr[(params.rank + r) % W])[fo + i] = o;
        }
    }
}

// Re-gather of a parameter group for the ZeRO-3 mode that does not keep a replica: copy table entries
// (owner rank, offset in that rank's bf16 shard buffer) -> offset in the local gathered buffer, plain P2P loads.
struct GatherTable {
    int n;
    int owner[MAX_SEGS];
    long long src_off[MAX_SEGS];
    long long dst_off[MAX_SEGS];
    long long numel[MAX_SEGS];
    int cta_begin[MAX_SEGS + 1];
};
__global__ void __launch_bounds__(256) zero_gather_segments_kernel(PeerTable shards, GatherTable t, __nv_bfloat16* __restrict__ dst) {
    int s = 0;
    while (s + 1 < t.n && int(blockIdx.x) >= t.cta_begin[s + 1]) ++s;
    const long long b = blockIdx.x - t.cta_begin[s], nb = t.cta_begin[s + 1] - t.cta_begin[s];
    if (nb <= 0) return;
    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(shards.ptr[t.owner[s]]) + t.src_off[s];
    __nv_bfloat16* out = dst + t.dst_off[s];
    const long long n = t.numel[s];
    const bool vec_ok = (t.src_off[s] % 8 == 0) && (t.dst_off[s] % 8 == 0);
    const long long nvec = vec_ok ? n / 8 : 0;
    const long long stride = nb * blockDim.x;
    for (long long i0 = b * blockDim.x + threadIdx.x; i0 < nvec; i0 += 4 * stride) {      // four 16-byte peer loads in flight
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i0 + u * stride < nvec) v[u] = __ldg(reinterpret_cast<const uint4*>(src) + i0 + u * stride);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i0 + u * stride < nvec) reinterpret_cast<uint4*>(out)[i0 + u * stride] = v[u];
    }
    for (long long i = nvec * 8 + b * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = src[i];
}

static PeerTable make_peers(void* const* ptrs, int world, int rank) {
    PeerTable t{};
    t.world = world; t.rank = rank;
    for (int r = 0; r < world && r < MAX_RANKS; ++r) t.ptr[r] = ptrs[r];
    return t;
}
static SegTable make_segs(int n, const long long* full_off, const long long* shard_off, const long long* numel, int ctas = 0) {
    SegTable s{};
    s.n = n;
    long long total = 0;
    for (int i = 0; i < n; ++i) { s.full_off[i] = full_off[i]; s.shard_off[i] = shard_off[i]; s.numel[i] = numel[i]; total += numel[i]; }
    // CTA ranges: segment i ends at the rounded share of the element prefix, every non-empty segment gets at
    // least one CTA and leaves one for each non-empty segment after it; the last one ends at `ctas`
    int given = 0, nonempty_after = 0;
    for (int i = 0; i < n; ++i) nonempty_after += numel[i] > 0;
    long long prefix = 0;
    for (int i = 0; i < n; ++i) {
        s.cta_begin[i] = given;
        if (numel[i] > 0 && ctas > 0) {
            --nonempty_after;
            prefix += numel[i];
            int end = int((long double)prefix / (long double)total * ctas + 0.5L);
            if (end > ctas - nonempty_after) end = ctas - nonempty_after;
            if (nonempty_after == 0) end = ctas;
            if (end < given + 1) end = given + 1;
            given = end;
        }
    }
    s.cta_begin[n] = given;
    return s;
}

}  // namespace pb

using namespace pb;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int pb_zero_max_segs() { return MAX_SEGS; }
extern "C" int pb_zero_max_ranks() { return MAX_RANKS; }
// Host-only: the CTA ranges that a launch over these segments would use (cta_begin[0..nseg]); returns the grid size.
extern "C" int pb_zero_cta_ranges(int nseg, const long long* numel, int ctas, int* cta_begin) {
    if (nseg > MAX_SEGS || nseg < 0) return -1;
    if (ctas < nseg) ctas = nseg;
    const SegTable sg = make_segs(nseg, numel, numel, numel, ctas);
    for (int i = 0; i <= nseg; ++i) cta_begin[i] = sg.cta_begin[i];
    return sg.cta_begin[nseg];
}

// How long a peer wait may spin before it gives up with PB_ERR_TIMEOUT_PEER. Passed to the kernels as an argument on
// every launch; the default is the compile-time budget of the other bounded waits (2 s).
static unsigned long long g_peer_wait_budget_ns = PB_WAIT_BUDGET_NS;
extern "C" int pb_set_peer_wait_budget_ns(long long ns) {
    if (ns <= 0) return -1;
    g_peer_wait_budget_ns = (unsigned long long)ns;
    return 0;
}
extern "C" long long pb_get_peer_wait_budget_ns() { return (long long)g_peer_wait_budget_ns; }

extern "C" int pb_peer_barrier(void* const* pad_ptrs, int world, int rank, int slot, int epoch, int* status, void* stream) {
    if (world > MAX_RANKS) return -1;
    peer_barrier_kernel<<<1, 32, 0, ST(stream)>>>(make_peers(pad_ptrs, world, rank), slot, epoch, status, g_peer_wait_budget_ns);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

extern "C" int pb_allreduce_scalars(void* const* flag_pads, void* const* data_pads, int world, int rank, int slot, int epoch,
                                    const float* in, float* out, int n, int* status, void* stream) {
    if (world > MAX_RANKS || n > 8) return -1;
    allreduce_scalars_kernel<<<1, 32, 0, ST(stream)>>>(make_peers(flag_pads, world, rank), make_peers(data_pads, world, rank), slot,
                                                       epoch, in, out, n, status, g_peer_wait_budget_ns);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

// sumsq_out (+)= sum of squares of the reduced, scaled shard values of these segments.
// partial: scratch of >= ctas floats.
extern "C" int pb_zero_reduce_grads(void* const* peer_grads, int world, int rank, int grad_fp32, int nseg,
                                    const long long* full_off, const long long* shard_off, const long long* numel,
                                    float* grad_shard, float scale, float* partial, float* sumsq_out, int accumulate, int ctas,
                                    void* stream) {
    if (world > MAX_RANKS || nseg > MAX_SEGS) return -1;
    PeerTable pt = make_peers(peer_grads, world, rank);
    if (ctas < nseg) ctas = nseg;
    SegTable sg = make_segs(nseg, full_off, shard_off, numel, ctas);
    ctas = sg.cta_begin[nseg];
    if (ctas <= 0) return 0;
    if (grad_fp32) zero_reduce_grads_kernel<float><<<ctas, 256, 0, ST(stream)>>>(pt, sg, grad_shard, scale, partial);
    else zero_reduce_grads_kernel<__nv_bfloat16><<<ctas, 256, 0, ST(stream)>>>(pt, sg, grad_shard, scale, partial);
    reduce_partials_kernel<<<1, 32, 0, ST(stream)>>>(partial, ctas, sumsq_out, accumulate);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

extern "C" int pb_zero_adamw_gather(void* const* peer_params, int world, int rank, int nseg, const long long* full_off,
                                    const long long* shard_off, const long long* numel, float* master, const float* grad_shard,
                                    float* m, float* v, float lr, float beta1, float beta2, float eps, float wd, int step,
                                    const float* gnorm_sq, float max_norm, int ctas, void* stream) {
    if (world > MAX_RANKS || nseg > MAX_SEGS) return -1;
    const float bc1 = 1.f - powf(beta1, float(step));
    const float bc2 = sqrtf(1.f - powf(beta2, float(step)));
    if (ctas < nseg) ctas = nseg;
    const SegTable sg = make_segs(nseg, full_off, shard_off, numel, ctas);
    if (sg.cta_begin[nseg] <= 0) return 0;
    zero_adamw_gather_kernel<<<sg.cta_begin[nseg], 256, 0, ST(stream)>>>(make_peers(peer_params, world, rank), sg, master, grad_shard, m, v,
                                                                         lr, beta1, beta2, eps, wd, bc1, bc2, gnorm_sq, max_norm);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

// dst[dst_off[i] ..) = rank owner[i]'s shard buffer [src_off[i] ..), numel[i] bf16 elements each.
extern "C" int pb_zero_gather_segments(void* const* peer_shards, int world, int rank, int nseg, const int* owner, const long long* src_off,
                                       const long long* dst_off, const long long* numel, void* dst, int ctas, void* stream) {
    if (world > MAX_RANKS || nseg > MAX_SEGS || nseg < 0) return -1;
    if (nseg == 0) return 0;
    GatherTable t{};
    t.n = nseg;
    if (ctas < nseg) ctas = nseg;
    const SegTable sg = make_segs(nseg, src_off, dst_off, numel, ctas);      // only its CTA split is used
    for (int i = 0; i < nseg; ++i) {
        if (owner[i] < 0 || owner[i] >= world) return -1;
        t.owner[i] = owner[i]; t.src_off[i] = src_off[i]; t.dst_off[i] = dst_off[i]; t.numel[i] = numel[i];
    }
    for (int i = 0; i <= nseg; ++i) t.cta_begin[i] = sg.cta_begin[i];
    if (sg.cta_begin[nseg] <= 0) return 0;
    zero_gather_segments_kernel<<<sg.cta_begin[nseg], 256, 0, ST(stream)>>>(make_peers(peer_shards, world, rank), t,
                                                                             reinterpret_cast<__nv_bfloat16*>(dst));
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}

extern "C" int pb_zero_push_params(void* const* peer_params, int world, int rank, int nseg, const long long* full_off,
                                   const long long* shard_off, const long long* numel, const float* master, int ctas, void* stream) {
    if (world > MAX_RANKS || nseg > MAX_SEGS) return -1;
    zero_push_params_kernel<<<ctas, 256, 0, ST(stream)>>>(make_peers(peer_params, world, rank),
                                                          make_segs(nseg, full_off, shard_off, numel), master);
    return cudaGetLastError() == cudaSuccess ? 0 : -30;
}
