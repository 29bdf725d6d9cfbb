// Exercises the host library (uint8 quantiser + TCP ring all-reduce) in one process so that it can be
// built with -fsanitize=address,undefined (and, separately, thread): odd sizes, tails, 1-element inputs,
// and a 3-rank ring over loopback with each rank on its own thread. Exit code 0 = all checks passed.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

extern "C" {
double pbh_sumsq(const float* x, int64_t n, int threads);
float pbh_uniform_8bit_quantize(const float* x, int64_t n, uint8_t* q, float* lut, int threads);
void pbh_dequant_add(float* dst, const uint8_t* q, const float* lut, int64_t n, int threads);
void pbh_dequant_set(float* dst, const uint8_t* q, const float* lut, int64_t n, int threads);
void* pbh_ring_create(int rank, int world, int nconn, int port, double timeout_s);
int pbh_ring_port(void* h);
int pbh_ring_connect(void* h, const char* next_host, int next_port);
int pbh_ring_allreduce(void* h, float* data, int64_t n, int quantize, int average, int threads);
void pbh_ring_destroy(void* h);
}

static int fails = 0;
#define CHECK(c) do { if (!(c)) { std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #c); ++fails; } } while (0)

static float frand(uint32_t& s) { s = s * 1664525u + 1013904223u; return float(int32_t(s >> 8) % 20001 - 10000) * 1e-4f; }

static void quantiser_cases() {
    const int64_t sizes[] = {1, 2, 7, 255, 256, 257, 4099, 100003};
    for (int64_t n : sizes)
        for (int threads : {1, 3, 8}) {
            uint32_t seed = uint32_t(n) * 77u + threads;
            std::vector<float> x(n), y(n, 0.f), z(n, 1.f);
            for (auto& v : x) v = frand(seed);
            std::vector<uint8_t> q(n);
            float lut[256];
            pbh_uniform_8bit_quantize(x.data(), n, q.data(), lut, threads);
            pbh_dequant_set(y.data(), q.data(), lut, n, threads);
            pbh_dequant_add(z.data(), q.data(), lut, n, threads);
            double err = 0, ref = 0;
            for (int64_t i = 0; i < n; ++i) {
                err += (x[i] - y[i]) * double(x[i] - y[i]);
                ref += x[i] * double(x[i]);
                CHECK(std::fabs(z[i] - (1.f + y[i])) < 1e-6f);
            }
            if (n > 256) CHECK(err <= 0.01 * ref + 1e-12);
            CHECK(std::fabs(pbh_sumsq(x.data(), n, threads) - ref) <= 1e-6 * (ref + 1e-12));
        }
}

static void ring_case(int world, int64_t n, int quantize) {
    std::vector<void*> h(world);
    for (int r = 0; r < world; ++r) { h[r] = pbh_ring_create(r, world, 2, 0, 20.0); CHECK(h[r] != nullptr); }
    std::vector<std::vector<float>> data(world, std::vector<float>(n));
    std::vector<double> want(n, 0.0);
    for (int r = 0; r < world; ++r) {
        uint32_t seed = 1234u + r;
        for (int64_t i = 0; i < n; ++i) { data[r][i] = frand(seed); want[i] += data[r][i]; }
    }
    std::vector<std::thread> th;
    std::vector<int> rc(world, -1);
    for (int r = 0; r < world; ++r)
        th.emplace_back([&, r] {
            if (pbh_ring_connect(h[r], "127.0.0.1", pbh_ring_port(h[(r + 1) % world])) != 0) return;
            rc[r] = pbh_ring_allreduce(h[r], data[r].data(), n, quantize, 0, 2);
        });
    for (auto& t : th) t.join();
    double err = 0, ref = 0;
    for (int r = 0; r < world; ++r) {
        CHECK(rc[r] == 0);
        for (int64_t i = 0; i < n; ++i) {
            if (r == 0) { err += (data[0][i] - want[i]) * (data[0][i] - want[i]); ref += want[i] * want[i]; }
            CHECK(data[r][i] == data[0][i]);          // every rank ends with the same bits
        }
    }
    CHECK(err <= (quantize ? 0.02 : 1e-10) * ref + 1e-12);
    for (int r = 0; r < world; ++r) pbh_ring_destroy(h[r]);
}

int main() {
    quantiser_cases();
    ring_case(3, 100003, 1);
    ring_case(3, 5, 1);          // fewer elements than ring chunks
    ring_case(2, 70001, 0);
    std::printf("host_sanitize: %d failure(s)\n", fails);
    return fails ? 1 : 0;
}
