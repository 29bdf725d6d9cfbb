// Host-side uint8 quantizer for pseudo-gradients (used by CPU ranks and by the cross-node TCP ring).
//
// Semantics follow the reference quantizer (src/zeroband/C/csrc/compression.cpp:9-125):
//   std   = ||x||_2 / sqrt(n - 1)           (no mean subtraction)
//   scale = 6 * std / 256
//   q[i]  = clamp(round_half_away(x[i] / scale) + 128, 0, 255)
//   lut[b] = mean of the x[i] that landed in bin b (0 for an empty bin)
// Differences by design: the work is split into fixed contiguous ranges whose partial sums are
// merged in range order, so the codebook is bit-reproducible for a given thread count (the
// reference merges thread-local sums under a mutex in arrival order), and the index-add /
// index-set dequantisers are actually multithreaded.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr int kBins = 256;
constexpr int kOffset = 128;
constexpr double kRangeSigmas = 6.0;

int pick_threads(int64_t n, int requested) {
    int hw = requested > 0 ? requested : int(std::thread::hardware_concurrency());
    if (hw < 1) hw = 1;
    const int64_t by_size = std::max<int64_t>(1, n / 65536);
    return int(std::min<int64_t>(hw, by_size));
}

template <typename Fn>
void parallel_ranges(int64_t n, int threads, Fn fn) {
    if (threads <= 1) {
        fn(0, int64_t(0), n);
        return;
    }
    std::vector<std::thread> pool;
    const int64_t per = (n + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const int64_t lo = std::min<int64_t>(n, t * per), hi = std::min<int64_t>(n, lo + per);
        pool.emplace_back([=] { fn(t, lo, hi); });
    }
    for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

// sum of squares in double, fixed-order merge
double pbh_sumsq(const float* x, int64_t n, int threads) {
    threads = pick_threads(n, threads);
    std::vector<double> part(threads, 0.0);
    parallel_ranges(n, threads, [&](int t, int64_t lo, int64_t hi) {
        double s = 0.0;
        for (int64_t i = lo; i < hi; ++i) s += double(x[i]) * double(x[i]);
        part[t] = s;
    });
    double s = 0.0;
    for (double p : part) s += p;
    return s;
}

// q[i] = clamp(round(x[i] * inv_scale) + zero_point, 0, 255)
void pbh_quantize_per_tensor_uint8(const float* x, int64_t n, float scale, int zero_point, uint8_t* q, int threads) {
    threads = pick_threads(n, threads);
    const float inv = 1.0f / scale;
    parallel_ranges(n, threads, [&](int, int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) {
            const int v = int(std::round(x[i] * inv)) + zero_point;
            q[i] = uint8_t(std::min(255, std::max(0, v)));
        }
    });
}

// lut[b] = mean{x[i] : q[i] == b}
void pbh_average_buckets(const float* x, const uint8_t* q, int64_t n, float* lut, int threads) {
    threads = pick_threads(n, threads);
    std::vector<double> sums(size_t(threads) * kBins, 0.0);
    std::vector<int64_t> cnts(size_t(threads) * kBins, 0);
    parallel_ranges(n, threads, [&](int t, int64_t lo, int64_t hi) {
        double* s = sums.data() + size_t(t) * kBins;
        int64_t* c = cnts.data() + size_t(t) * kBins;
        for (int64_t i = lo; i < hi; ++i) {
            s[q[i]] += x[i];
            c[q[i]] += 1;
        }
    });
    for (int b = 0; b < kBins; ++b) {
        double s = 0.0;
        int64_t c = 0;
        for (int t = 0; t < threads; ++t) {
            s += sums[size_t(t) * kBins + b];
            c += cnts[size_t(t) * kBins + b];
        }
        lut[b] = c > 0 ? float(s / double(c)) : 0.0f;
    }
}

// full quantizer: returns the scale used
float pbh_uniform_8bit_quantize(const float* x, int64_t n, uint8_t* q, float* lut, int threads) {
    const double ss = pbh_sumsq(x, n, threads);
    const double stdv = n > 1 ? std::sqrt(ss / double(n - 1)) : std::sqrt(ss);
    float scale = float(kRangeSigmas * stdv / kBins);
    if (!(scale > 0.0f) || !std::isfinite(scale)) scale = 1.0f;   // all-zero (e.g. a joiner's fake pseudo-gradient)
    pbh_quantize_per_tensor_uint8(x, n, scale, kOffset, q, threads);
    pbh_average_buckets(x, q, n, lut, threads);
    return scale;
}

// dst[i] += lut[q[i]]
void pbh_dequant_add(float* dst, const uint8_t* q, const float* lut, int64_t n, int threads) {
    threads = pick_threads(n, threads);
    parallel_ranges(n, threads, [&](int, int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) dst[i] += lut[q[i]];
    });
}

// dst[i] = lut[q[i]]
void pbh_dequant_set(float* dst, const uint8_t* q, const float* lut, int64_t n, int threads) {
    threads = pick_threads(n, threads);
    parallel_ranges(n, threads, [&](int, int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) dst[i] = lut[q[i]];
    });
}

void pbh_scale(float* x, int64_t n, float s, int threads) {
    threads = pick_threads(n, threads);
    parallel_ranges(n, threads, [&](int, int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) x[i] *= s;
    });
}

}  // extern "C"
