// Cross-node pseudo-gradient all-reduce over plain TCP sockets: a pipelined ring with optional
// uint8 quantisation and fp32 accumulation. No gloo, no MPI: each rank listens on one port,
// connects to its successor (several parallel sockets per link) and accepts from its predecessor.
//
// What the reference does (src/zeroband/C/csrc/collectives.cpp:76-230): 2W chunks, two interleaved
// rings of c10d send/recv, every hop re-quantises, and in the all-gather phase forwarders re-quantise
// an already dequantised chunk, so ranks do not end bit-identical. This implementation:
//   * reduce-scatter: W-1 hops; every hop quantises its current partial sum (uint8 + 256-entry fp32
//     codebook per sub-chunk), the receiver dequantises and accumulates in fp32;
//   * the owner quantises its reduced chunk ONCE; the all-gather forwards those bytes verbatim, and
//     the owner itself adopts the dequantised values, so every rank ends with identical bits;
//   * each chunk is cut into sub-chunks that flow through a sender thread (quantise -> write) while
//     the caller thread reads and dequantises, so arithmetic overlaps the wire in both directions;
//   * a link is `nconn` sockets; sub-chunk i travels on socket i % nconn (parallel TCP streams);
//   * tensors of any length work (chunks are ceil-divided, tails may be empty);
//   * every socket has send/receive timeouts; any failure returns a negative code (never blocks
//     forever) and poisons the ring so the caller rebuilds it — this feeds DiLoCo's retry path.
#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

extern "C" {
float pbh_uniform_8bit_quantize(const float* x, int64_t n, uint8_t* q, float* lut, int threads);
void pbh_dequant_add(float* dst, const uint8_t* q, const float* lut, int64_t n, int threads);
void pbh_dequant_set(float* dst, const uint8_t* q, const float* lut, int64_t n, int threads);
}

namespace {

constexpr int kErrSocket = -1, kErrConnect = -2, kErrIO = -3, kErrPoisoned = -4, kErrArg = -5;
constexpr int64_t kSubChunk = 1 << 20;   // elements per pipelined sub-chunk

struct Ring {
    int rank = 0, world = 1, nconn = 1;
    int listen_fd = -1;
    int port = 0;
    std::vector<int> next_fds, prev_fds;
    double timeout_s = 30.0;
    std::atomic<bool> poisoned{false};
    std::atomic<int> fault_after_bytes{-1};   // test hook: fail a write once this many bytes went out
    int64_t bytes_sent = 0;
};

void set_timeouts(int fd, double seconds) {
    timeval tv;
    tv.tv_sec = long(seconds);
    tv.tv_usec = long((seconds - double(tv.tv_sec)) * 1e6);
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    int buf = 8 << 20;
    setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
    setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
}

bool write_all(Ring* r, int fd, const void* p, size_t n) {
    const char* c = static_cast<const char*>(p);
    while (n > 0) {
        const int lim = r->fault_after_bytes.load();
        if (lim >= 0 && r->bytes_sent >= lim) {   // injected link failure
            shutdown(fd, SHUT_RDWR);
            return false;
        }
        ssize_t k = ::send(fd, c, n, MSG_NOSIGNAL);
        if (k <= 0) {
            if (k < 0 && errno == EINTR) continue;
            return false;
        }
        c += k;
        n -= size_t(k);
        r->bytes_sent += k;
    }
    return true;
}

bool read_all(int fd, void* p, size_t n) {
    char* c = static_cast<char*>(p);
    while (n > 0) {
        ssize_t k = ::recv(fd, c, n, 0);
        if (k <= 0) {
            if (k < 0 && errno == EINTR) continue;
            return false;
        }
        c += k;
        n -= size_t(k);
    }
    return true;
}

struct ChunkRange { int64_t lo, hi; };
ChunkRange chunk_of(int64_t n, int world, int c) {
    const int64_t per = (n + world - 1) / world;
    const int64_t lo = std::min<int64_t>(n, int64_t(c) * per);
    return {lo, std::min<int64_t>(n, lo + per)};
}

}  // namespace

extern "C" {

// Create the ring endpoint and start listening. port = 0 picks a free port. Returns handle or null.
void* pbh_ring_create(int rank, int world, int nconn, int port, double timeout_s) {
    if (world < 1 || rank < 0 || rank >= world || nconn < 1 || nconn > 16) return nullptr;
    Ring* r = new Ring();
    r->rank = rank; r->world = world; r->nconn = nconn; r->timeout_s = timeout_s;
    r->listen_fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (r->listen_fd < 0) { delete r; return nullptr; }
    int one = 1;
    setsockopt(r->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_addr.s_addr = htonl(INADDR_ANY);
    addr.sin_port = htons(uint16_t(port));
    if (::bind(r->listen_fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(r->listen_fd, 64) != 0) {
        ::close(r->listen_fd);
        delete r;
        return nullptr;
    }
    socklen_t len = sizeof(addr);
    getsockname(r->listen_fd, reinterpret_cast<sockaddr*>(&addr), &len);
    r->port = ntohs(addr.sin_port);
    timeval tv;   // accept() must not block forever either
    tv.tv_sec = long(timeout_s);
    tv.tv_usec = 0;
    setsockopt(r->listen_fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    return r;
}

int pbh_ring_port(void* h) { return h ? static_cast<Ring*>(h)->port : -1; }

// Connect to the successor at host:port and accept the predecessor's sockets. Every rank calls this
// after all ranks have published their listening address.
int pbh_ring_connect(void* h, const char* next_host, int next_port) {
    Ring* r = static_cast<Ring*>(h);
    if (!r) return kErrArg;
    if (r->world == 1) return 0;
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    const std::string port_s = std::to_string(next_port);
    if (getaddrinfo(next_host, port_s.c_str(), &hints, &res) != 0 || !res) return kErrConnect;
    int rc = 0;
    for (int i = 0; i < r->nconn && rc == 0; ++i) {
        int fd = ::socket(AF_INET, SOCK_STREAM, 0);
        if (fd < 0) { rc = kErrSocket; break; }
        set_timeouts(fd, r->timeout_s);
        bool ok = false;
        for (int attempt = 0; attempt < 50 && !ok; ++attempt) {   // the peer may not be listening yet
            ok = ::connect(fd, res->ai_addr, res->ai_addrlen) == 0;
            if (!ok) usleep(100000);
        }
        if (!ok) { ::close(fd); rc = kErrConnect; break; }
        const int32_t hello[2] = {r->rank, i};
        if (!write_all(r, fd, hello, sizeof(hello))) { ::close(fd); rc = kErrIO; break; }
        r->next_fds.push_back(fd);
    }
    freeaddrinfo(res);
    if (rc) return rc;
    r->prev_fds.assign(r->nconn, -1);
    for (int i = 0; i < r->nconn; ++i) {
        int fd = ::accept(r->listen_fd, nullptr, nullptr);
        if (fd < 0) return kErrConnect;
        set_timeouts(fd, r->timeout_s);
        int32_t hello[2];
        if (!read_all(fd, hello, sizeof(hello)) || hello[1] < 0 || hello[1] >= r->nconn) { ::close(fd); return kErrIO; }
        r->prev_fds[hello[1]] = fd;
    }
    r->bytes_sent = 0;
    return 0;
}

void pbh_ring_destroy(void* h) {
    Ring* r = static_cast<Ring*>(h);
    if (!r) return;
    for (int fd : r->next_fds) if (fd >= 0) ::close(fd);
    for (int fd : r->prev_fds) if (fd >= 0) ::close(fd);
    if (r->listen_fd >= 0) ::close(r->listen_fd);
    delete r;
}

// Test hook: make this rank's outgoing link fail after `bytes` more bytes (-1 disables).
void pbh_ring_inject_fault(void* h, int bytes) {
    Ring* r = static_cast<Ring*>(h);
    if (r) r->fault_after_bytes.store(bytes < 0 ? -1 : int(r->bytes_sent + bytes));
}

// In-place all-reduce (sum, or mean when `average`) of data[0..n). quantize: 0 = fp32 on the wire,
// 1 = uint8 + codebook on the wire with fp32 accumulation. Returns 0 or a negative error code.
int pbh_ring_allreduce(void* h, float* data, int64_t n, int quantize, int average, int threads) {
    Ring* r = static_cast<Ring*>(h);
    if (!r || n < 0) return kErrArg;
    if (r->poisoned.load()) return kErrPoisoned;
    const int W = r->world, me = r->rank;
    if (W == 1 || n == 0) return 0;
    std::atomic<bool> failed{false};

    // one hop: send chunk `sc` to the successor while receiving chunk `rc` from the predecessor.
    // mode 0: receiver accumulates (reduce-scatter). mode 1: receiver overwrites (all-gather).
    // In all-gather with quantisation, payloads are forwarded verbatim from `fwd_q`/`fwd_lut` storage.
    struct Packed { std::vector<uint8_t> q; std::vector<float> lut; };   // per chunk: quantised bytes + one codebook per sub-chunk
    std::vector<Packed> packed(W);

    auto hop = [&](int sc, int rcv, int mode) {
        const ChunkRange s = chunk_of(n, W, sc), g = chunk_of(n, W, rcv);
        const int64_t sn = s.hi - s.lo, gn = g.hi - g.lo;
        const int64_t s_sub = (sn + kSubChunk - 1) / kSubChunk, g_sub = (gn + kSubChunk - 1) / kSubChunk;
        std::thread sender([&] {
            std::vector<uint8_t> qbuf;
            float lut[256];
            for (int64_t i = 0; i < s_sub && !failed.load(); ++i) {
                const int64_t lo = s.lo + i * kSubChunk, cnt = std::min<int64_t>(kSubChunk, s.hi - lo);
                const int fd = r->next_fds[i % r->nconn];
                bool ok;
                if (!quantize) {
                    ok = write_all(r, fd, data + lo, size_t(cnt) * 4);
                } else if (mode == 1) {   // forward the owner's bytes untouched
                    ok = write_all(r, fd, packed[sc].lut.data() + i * 256, 1024) &&
                         write_all(r, fd, packed[sc].q.data() + i * kSubChunk, size_t(cnt));
                } else {
                    qbuf.resize(size_t(cnt));
                    pbh_uniform_8bit_quantize(data + lo, cnt, qbuf.data(), lut, threads);
                    ok = write_all(r, fd, lut, 1024) && write_all(r, fd, qbuf.data(), size_t(cnt));
                }
                if (!ok) failed.store(true);
            }
        });
        std::vector<float> fbuf;
        std::vector<uint8_t> qbuf;
        float lut[256];
        if (quantize && mode == 1) {
            packed[rcv].q.resize(size_t(gn));
            packed[rcv].lut.resize(size_t(g_sub) * 256);
        }
        for (int64_t i = 0; i < g_sub && !failed.load(); ++i) {
            const int64_t lo = g.lo + i * kSubChunk, cnt = std::min<int64_t>(kSubChunk, g.hi - lo);
            const int fd = r->prev_fds[i % r->nconn];
            bool ok;
            if (!quantize) {
                if (mode == 1) {
                    ok = read_all(fd, data + lo, size_t(cnt) * 4);
                } else {
                    fbuf.resize(size_t(cnt));
                    ok = read_all(fd, fbuf.data(), size_t(cnt) * 4);
                    if (ok) for (int64_t k = 0; k < cnt; ++k) data[lo + k] += fbuf[k];
                }
            } else if (mode == 1) {
                uint8_t* qdst = packed[rcv].q.data() + i * kSubChunk;
                float* ldst = packed[rcv].lut.data() + i * 256;
                ok = read_all(fd, ldst, 1024) && read_all(fd, qdst, size_t(cnt));
                if (ok) pbh_dequant_set(data + lo, qdst, ldst, cnt, threads);
            } else {
                qbuf.resize(size_t(cnt));
                ok = read_all(fd, lut, 1024) && read_all(fd, qbuf.data(), size_t(cnt));
                if (ok) pbh_dequant_add(data + lo, qbuf.data(), lut, cnt, threads);
            }
            if (!ok) failed.store(true);
        }
        sender.join();
    };

    // reduce-scatter: after W-1 hops rank `me` owns the full sum of chunk (me + 1) % W
    for (int step = 0; step < W - 1 && !failed.load(); ++step)
        hop((me - step + W) % W, (me - step - 1 + W) % W, 0);
    const int own = (me + 1) % W;
    if (!failed.load()) {
        const ChunkRange o = chunk_of(n, W, own);
        const int64_t on = o.hi - o.lo;
        if (average) for (int64_t k = o.lo; k < o.hi; ++k) data[k] /= float(W);
        if (quantize) {   // quantise once; the owner adopts the values everybody else will see
            const int64_t subs = (on + kSubChunk - 1) / kSubChunk;
            packed[own].q.resize(size_t(on));
            packed[own].lut.resize(size_t(subs) * 256);
            for (int64_t i = 0; i < subs; ++i) {
                const int64_t lo = o.lo + i * kSubChunk, cnt = std::min<int64_t>(kSubChunk, o.hi - lo);
                pbh_uniform_8bit_quantize(data + lo, cnt, packed[own].q.data() + i * kSubChunk, packed[own].lut.data() + i * 256, threads);
                pbh_dequant_set(data + lo, packed[own].q.data() + i * kSubChunk, packed[own].lut.data() + i * 256, cnt, threads);
            }
        }
    }
    // all-gather: circulate the owned chunks
    for (int step = 0; step < W - 1 && !failed.load(); ++step)
        hop((own - step + W) % W, (own - step - 1 + W) % W, 1);
    if (failed.load()) {
        r->poisoned.store(true);
        return kErrIO;
    }
    return 0;
}

// Throughput probe used for ring ordering: push `bytes` to the successor link and time it. Both ends
// of a link call it (sender side returns seconds, receiver drains). Returns < 0 on error.
double pbh_ring_probe(void* h, int64_t bytes) {
    Ring* r = static_cast<Ring*>(h);
    if (!r || r->world == 1) return 0.0;
    std::vector<char> buf(1 << 20, 1);
    std::atomic<bool> failed{false};
    timeval t0, t1;
    gettimeofday(&t0, nullptr);
    std::thread sender([&] {
        for (int64_t sent = 0; sent < bytes && !failed.load(); sent += int64_t(buf.size()))
            if (!write_all(r, r->next_fds[0], buf.data(), buf.size())) failed.store(true);
    });
    std::vector<char> in(1 << 20);
    for (int64_t got = 0; got < bytes && !failed.load(); got += int64_t(in.size()))
        if (!read_all(r->prev_fds[0], in.data(), in.size())) failed.store(true);
    sender.join();
    gettimeofday(&t1, nullptr);
    if (failed.load()) { r->poisoned.store(true); return -1.0; }
    return double(t1.tv_sec - t0.tv_sec) + double(t1.tv_usec - t0.tv_usec) * 1e-6;
}

}  // extern "C"
