// megray_bench: collective benchmark over the public C++ interface.
//
// Same job and the same short flags as the reference's `performance` tool
// (reference test/performance.cpp:438-495: -d devices, -I master ip, -P port, -n nodes,
// -r node rank, -e backends, -f functions, -s sizes, -w warm-up, -i iterations), but:
//   * every call is timed on the device with CUDA events and the reported time is the
//     MAX over ranks (the reference times on the host and reports one rank's view);
//   * bus bandwidth is reported next to the reference's "speed" (bytes of the per-rank
//     unit over time): all_reduce x 2(n-1)/n, all_gather / reduce_scatter / all_to_all /
//     gather / scatter x (n-1), broadcast / reduce / send_recv x 1;
//   * any list of dtypes (-t float32,bfloat16 | all) and reduce ops (-o sum,max | all), sizes
//     given in bytes or as a doubling range (-s 1K:1G), JSON lines with -j;
//   * buffers hold seeded data (uniform[-1,1] floats, integers in [-100,100], a different
//     stream per rank) and, with -c, every result is checked against values computed on the host;
//   * one communicator group per backend serves all functions, dtypes, ops and sizes.
// Ranks are threads of this process, one GPU each (as the reference's tests and benchmark
// drive them).  Because it uses only the interface shared with the reference, this file
// also compiles against the reference's own headers and objects (-DMEGRAY_BENCH_REFERENCE):
// that build is the like-for-like baseline.
#include <cuda_runtime.h>

#include <chrono>
#include <getopt.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <functional>
#include <map>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "megray.h"

using namespace MegRay;

namespace {

struct BenchOptions {
    int devices = 2;
    std::string master_ip = "127.0.0.1";
    int port = 0;
    int nodes = 1, node_rank = 0;
    std::vector<std::string> backends;
    std::vector<std::string> funcs;
    std::vector<size_t> sizes;
    int warmup = 20, iters = 50;
    std::vector<std::string> dtypes;
    std::vector<std::string> ops;
    bool json = false;
    bool check = false;
    bool heap = false;  // NVL backend: buffers from the symmetric heap (zero-copy / NVSwitch kernels)
    bool reg = false;   // NVL backend: cudaMalloc buffers registered with the communicator (zero-copy)
    bool host = false;  // shm backend with CPU ranks: host buffers, wall-clock timing, no GPU needed
    bool phases = false;  // NVL backend: report where the time of the last call of each case went
};

const char* kAllFuncs[] = {"send_recv", "scatter", "gather", "all_to_all", "all_gather",
                           "all_reduce", "reduce_scatter", "broadcast", "reduce"};

enum Kind { K_INT, K_UINT, K_F16, K_BF16, K_F32, K_F64 };
struct DTypeInfo {
    const char* name;
    DType dtype;
    size_t size;
    Kind kind;
};
const DTypeInfo kDTypes[] = {
        {"int8", MEGRAY_INT8, 1, K_INT},       {"uint8", MEGRAY_UINT8, 1, K_UINT},     {"int32", MEGRAY_INT32, 4, K_INT},
        {"uint32", MEGRAY_UINT32, 4, K_UINT},  {"int64", MEGRAY_INT64, 8, K_INT},      {"uint64", MEGRAY_UINT64, 8, K_UINT},
        {"float16", MEGRAY_FLOAT16, 2, K_F16}, {"float32", MEGRAY_FLOAT32, 4, K_F32},  {"float64", MEGRAY_FLOAT64, 8, K_F64},
#ifndef MEGRAY_BENCH_REFERENCE
        {"bfloat16", MEGRAY_BFLOAT16, 2, K_BF16},
#endif
};

size_t parse_size(const std::string& s) {
    char* end = nullptr;
    double v = strtod(s.c_str(), &end);
    if (end && (*end == 'K' || *end == 'k')) v *= 1024.0;
    if (end && (*end == 'M' || *end == 'm')) v *= 1024.0 * 1024.0;
    if (end && (*end == 'G' || *end == 'g')) v *= 1024.0 * 1024.0 * 1024.0;
    return static_cast<size_t>(v);
}

std::vector<std::string> split(const std::string& s, char sep) {
    std::vector<std::string> out;
    size_t b = 0;
    while (b <= s.size()) {
        size_t e = s.find(sep, b);
        if (e == std::string::npos) e = s.size();
        if (e > b) out.push_back(s.substr(b, e - b));
        b = e + 1;
    }
    return out;
}

// A reusable barrier for the rank threads.
class ThreadBarrier {
public:
    explicit ThreadBarrier(int n) : m_n(n) {}
    void wait() {
        std::unique_lock<std::mutex> lk(m_mu);
        const uint64_t gen = m_gen;
        if (++m_count == m_n) {
            m_count = 0;
            ++m_gen;
            m_cv.notify_all();
        } else {
            m_cv.wait(lk, [&] { return m_gen != gen; });
        }
    }

private:
    int m_n, m_count = 0;
    uint64_t m_gen = 0;
    std::mutex m_mu;
    std::condition_variable m_cv;
};

double bus_factor(const std::string& f, int n) {
    if (f == "all_reduce") return 2.0 * (n - 1) / n;
    if (f == "all_gather" || f == "reduce_scatter" || f == "all_to_all" || f == "gather" || f == "scatter")
        return static_cast<double>(n - 1);
    return 1.0;
}

bool is_reducing(const std::string& f) { return f == "all_reduce" || f == "reduce_scatter" || f == "reduce"; }

Backend backend_of(const std::string& name) {
    if (name == "nccl" || name == "NCCL") return MEGRAY_NCCL;
    if (name == "shm" || name == "SHM") return MEGRAY_SHM;
#ifndef MEGRAY_BENCH_REFERENCE
    if (name == "nvl" || name == "NVL") return MEGRAY_NVL;
#endif
    if (name == "ucx" || name == "UCX") return MEGRAY_UCX;
    return MEGRAY_RCCL;
}

#define CK(expr)                                                                      \
    do {                                                                              \
        cudaError_t e_ = (expr);                                                      \
        if (e_ != cudaSuccess) {                                                      \
            fprintf(stderr, "cuda error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
            exit(1);                                                                  \
        }                                                                             \
    } while (0)

// ------------------------------------------------------------------ seeded data and the host check
// Every rank's input is one 1 MiB block of seeded values repeated over the buffer; the host keeps
// all ranks' blocks (as doubles) so that any output element can be predicted.
constexpr size_t kPatternBytes = 1u << 20;

uint16_t f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000;
    int e = static_cast<int>((x >> 23) & 0xff) - 127 + 15;
    uint32_t m = x & 0x7fffff;
    if (e <= 0) {
        if (e < -10) return static_cast<uint16_t>(sign);
        m |= 0x800000;
        const int shift = 14 - e;
        uint32_t r = m >> shift;
        if ((m >> (shift - 1)) & 1) r += 1;
        return static_cast<uint16_t>(sign | r);
    }
    if (e >= 31) return static_cast<uint16_t>(sign | 0x7c00);
    uint32_t r = (static_cast<uint32_t>(e) << 10) | (m >> 13);
    if (m & 0x1000) r += 1;
    return static_cast<uint16_t>(sign | r);
}
float f16_to_f32(uint16_t h) {
    const uint32_t sign = (h & 0x8000u) << 16;
    const int e = (h >> 10) & 0x1f;
    const uint32_t m = h & 0x3ff;
    if (e == 0) return (sign ? -1.f : 1.f) * ldexpf(static_cast<float>(m), -24);
    if (e == 31) return sign ? -INFINITY : INFINITY;
    const uint32_t x = sign | (static_cast<uint32_t>(e - 15 + 127) << 23) | (m << 13);
    float f;
    memcpy(&f, &x, 4);
    return f;
}
uint16_t f32_to_bf16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    x += 0x7fff + ((x >> 16) & 1);
    return static_cast<uint16_t>(x >> 16);
}
float bf16_to_f32(uint16_t b) {
    const uint32_t x = static_cast<uint32_t>(b) << 16;
    float f;
    memcpy(&f, &x, 4);
    return f;
}

// Fills `bytes` (one pattern block) for `rank` and returns the values as doubles.
std::vector<double> make_pattern(const DTypeInfo& dt, int rank, std::vector<char>* bytes) {
    const size_t count = kPatternBytes / dt.size;
    bytes->assign(kPatternBytes, 0);
    std::vector<double> vals(count);
    std::mt19937 gen(1234567u + 1000u * static_cast<unsigned>(rank) + static_cast<unsigned>(dt.dtype));
    std::uniform_real_distribution<float> uni(-1.f, 1.f);
    std::uniform_int_distribution<int> ints(-100, 100), uints(0, 100);
    for (size_t i = 0; i < count; ++i) {
        char* p = bytes->data() + i * dt.size;
        switch (dt.kind) {
            case K_F32: { float v = uni(gen); memcpy(p, &v, 4); vals[i] = v; break; }
            case K_F64: { double v = uni(gen); memcpy(p, &v, 8); vals[i] = v; break; }
            case K_F16: { uint16_t h = f32_to_f16(uni(gen)); memcpy(p, &h, 2); vals[i] = f16_to_f32(h); break; }
            case K_BF16: { uint16_t h = f32_to_bf16(uni(gen)); memcpy(p, &h, 2); vals[i] = bf16_to_f32(h); break; }
            case K_INT: {
                // (int8 sums of 8 values in [-100, 100] wrap; keep 8-bit inputs small instead)
                const int v = dt.size == 1 ? ints(gen) / 8 : ints(gen);
                if (dt.size == 1) { int8_t x = static_cast<int8_t>(v); memcpy(p, &x, 1); }
                else if (dt.size == 4) { int32_t x = v; memcpy(p, &x, 4); }
                else { int64_t x = v; memcpy(p, &x, 8); }
                vals[i] = v;
                break;
            }
            default: {
                const int v = dt.size == 1 ? uints(gen) / 8 : uints(gen);
                if (dt.size == 1) { uint8_t x = static_cast<uint8_t>(v); memcpy(p, &x, 1); }
                else if (dt.size == 4) { uint32_t x = static_cast<uint32_t>(v); memcpy(p, &x, 4); }
                else { uint64_t x = static_cast<uint64_t>(v); memcpy(p, &x, 8); }
                vals[i] = v;
            }
        }
    }
    return vals;
}

double read_value(const DTypeInfo& dt, const char* p) {
    switch (dt.kind) {
        case K_F32: { float v; memcpy(&v, p, 4); return v; }
        case K_F64: { double v; memcpy(&v, p, 8); return v; }
        case K_F16: { uint16_t h; memcpy(&h, p, 2); return f16_to_f32(h); }
        case K_BF16: { uint16_t h; memcpy(&h, p, 2); return bf16_to_f32(h); }
        case K_INT:
            if (dt.size == 1) { int8_t x; memcpy(&x, p, 1); return x; }
            if (dt.size == 4) { int32_t x; memcpy(&x, p, 4); return x; }
            { int64_t x; memcpy(&x, p, 8); return static_cast<double>(x); }
        default:
            if (dt.size == 1) { uint8_t x; memcpy(&x, p, 1); return x; }
            if (dt.size == 4) { uint32_t x; memcpy(&x, p, 4); return x; }
            { uint64_t x; memcpy(&x, p, 8); return static_cast<double>(x); }
    }
}

double tolerance(const DTypeInfo& dt, int n) {
    switch (dt.kind) {
        case K_F32: return 4e-6 * n;
        case K_F64: return 1e-13 * n;
        case K_F16: return 4e-3 * n;   // a library may round every pairwise sum to the 16-bit type
        case K_BF16: return 3e-2 * n;
        default: return 0.0;
    }
}

// ------------------------------------------------------------------ one backend: all measurements
struct Shared {
    ThreadBarrier bar;
    std::vector<double> times;
    std::vector<int> bad;
    std::atomic<bool> init_ok{true};
    // every rank's pattern of the current dtype, as doubles
    std::vector<std::vector<double>> pattern;
    explicit Shared(int n) : bar(n), times(n, 0.0), bad(n, 0), pattern(n) {}
};

void run_backend(const BenchOptions& o, const std::string& bname, Backend backend, int port) {
    const int n = o.devices;
    Shared sh(n);
    size_t max_unit = 0;
    for (size_t s : o.sizes) max_unit = std::max(max_unit, s);
    std::vector<const DTypeInfo*> dts;
    for (const auto& name : o.dtypes)
        for (const auto& d : kDTypes)
            if (name == d.name) dts.push_back(&d);
    std::vector<std::thread> threads;
    for (int r = 0; r < n; ++r) {
        threads.emplace_back([&, r] {
#ifndef MEGRAY_BENCH_REFERENCE
            const bool host = o.host && backend == MEGRAY_SHM;
#else
            const bool host = false;
#endif
            cudaStream_t stream = nullptr;
            std::shared_ptr<Context> ctx;
            if (!host) {
                CK(cudaSetDevice(r));
                CK(cudaStreamCreate(&stream));
                ctx = CudaContext::make(stream);
            }
#ifndef MEGRAY_BENCH_REFERENCE
            else {
                ctx = HostContext::make();
            }
#endif
            std::shared_ptr<Communicator> comm;
            try {
                comm = get_communicator(static_cast<uint32_t>(n), static_cast<uint32_t>(r), backend);
            } catch (const std::exception& e) {
                if (r == 0) fprintf(stderr, "backend unavailable: %s\n", e.what());
                sh.init_ok = false;
            }
            if (comm && comm->init(o.master_ip.c_str(), port) != MEGRAY_OK) sh.init_ok = false;
            sh.bar.wait();
            if (!sh.init_ok.load()) return;
            // one pair of buffers, sized for the widest operation at the largest size
            const size_t cap = std::max<size_t>(max_unit, 64) * n + 256;
            char *in = nullptr, *out = nullptr;
            bool from_heap = false;
#ifndef MEGRAY_BENCH_REFERENCE
            if (o.heap && backend == MEGRAY_NVL) {
                NvlInterface* nvl = as_nvl(comm.get());
                in = static_cast<char*>(nvl->sym_alloc(cap, nullptr));
                out = static_cast<char*>(nvl->sym_alloc(cap, nullptr));
                from_heap = true;
                if (in == nullptr || out == nullptr) {
                    fprintf(stderr, "symmetric heap too small for these sizes: raise MEGRAY_HEAP_MB\n");
                    exit(1);
                }
            }
#endif
            if (host) {
                in = static_cast<char*>(malloc(cap));
                out = static_cast<char*>(malloc(cap));
            } else if (!from_heap) {
                CK(cudaMalloc(&in, cap));
                CK(cudaMalloc(&out, cap));
            }
#ifndef MEGRAY_BENCH_REFERENCE
            bool registered = false;
            if (!from_heap && o.reg && backend == MEGRAY_NVL) {
                NvlInterface* nvl = as_nvl(comm.get());
                const Status s1 = nvl->register_buffer(in, cap);
                const Status s2 = nvl->register_buffer(out, cap);
                registered = s1 == MEGRAY_OK && s2 == MEGRAY_OK;
                if (!registered && r == 0)
                    fprintf(stderr, "buffers could not be registered: staged paths\n");
            }
#endif
            cudaEvent_t e0 = nullptr, e1 = nullptr;
            if (!host) {
                CK(cudaEventCreate(&e0));
                CK(cudaEventCreate(&e1));
            }
            const uint32_t root = 0;
            std::vector<char> block, window;
            for (const DTypeInfo* dtp : dts) {
                const DTypeInfo& dt = *dtp;
                // this rank's pattern block, repeated over the input buffer
                sh.pattern[r] = make_pattern(dt, r, &block);
                if (host) {
                    for (size_t off = 0; off < cap; off += kPatternBytes)
                        memcpy(in + off, block.data(), std::min(kPatternBytes, cap - off));
                } else {
                    CK(cudaMemcpy(in, block.data(), std::min(kPatternBytes, cap), cudaMemcpyHostToDevice));
                    for (size_t done = kPatternBytes; done < cap; done *= 2)
                        CK(cudaMemcpy(in + done, in, std::min(done, cap - done), cudaMemcpyDeviceToDevice));
                }
                sh.bar.wait();
                for (const std::string& func : o.funcs) {
                    std::vector<std::string> ops = is_reducing(func) ? o.ops : std::vector<std::string>{"-"};
                    for (const std::string& opname : ops) {
                        const ReduceOp op = opname == "max" ? MEGRAY_MAX : opname == "min" ? MEGRAY_MIN : MEGRAY_SUM;
                        for (size_t size : o.sizes) {
                            const size_t len = std::max<size_t>(1, size / dt.size);
                            auto call = [&]() -> Status {
                                if (func == "all_reduce") return comm->all_reduce(in, out, len, dt.dtype, op, ctx);
                                if (func == "all_gather") return comm->all_gather(in, out, len, dt.dtype, ctx);
                                if (func == "reduce_scatter") return comm->reduce_scatter(in, out, len, dt.dtype, op, ctx);
                                if (func == "all_to_all") return comm->all_to_all(in, out, len, dt.dtype, ctx);
                                if (func == "broadcast") return comm->broadcast(in, out, len, dt.dtype, root, ctx);
                                if (func == "reduce") return comm->reduce(in, out, len, dt.dtype, op, root, ctx);
                                if (func == "gather") return comm->gather(in, out, len, dt.dtype, root, ctx);
                                if (func == "scatter") return comm->scatter(in, out, len, dt.dtype, root, ctx);
                                if (func == "send_recv") {
                                    if (r == 0) return comm->send(in, len, dt.dtype, 1, ctx);
                                    if (r == 1) return comm->recv(out, len, dt.dtype, 0, ctx);
                                    return MEGRAY_OK;
                                }
                                return MEGRAY_INVALID_ARGUMENT;
                            };
                            // fewer repetitions for very large messages keep the sweep short
                            const bool big = size >= (64u << 20);
                            const int iters = big ? std::max(3, o.iters / 10) : o.iters;
                            const int warm = big ? std::max(2, o.warmup / 10) : o.warmup;
                            bool ok = true;
#ifndef MEGRAY_BENCH_REFERENCE
                            const CommStats st0 = comm->stats();
#endif
                            if (o.check && !host) CK(cudaMemsetAsync(out, 0xa5, std::min(cap, len * dt.size * n), stream));
                            for (int i = 0; i < warm && ok; ++i) ok = call() == MEGRAY_OK;
                            if (host) {
                                // CPU ranks: the calls are synchronous, wall clock between two thread barriers
                                sh.bar.wait();
                                const auto t0 = std::chrono::steady_clock::now();
                                for (int i = 0; i < iters && ok; ++i) ok = call() == MEGRAY_OK;
                                const auto t1 = std::chrono::steady_clock::now();
                                sh.times[r] = std::chrono::duration<double, std::micro>(t1 - t0).count() / iters;
                            } else {
                                CK(cudaStreamSynchronize(stream));
                                sh.bar.wait();
                                CK(cudaEventRecord(e0, stream));
                                for (int i = 0; i < iters && ok; ++i) ok = call() == MEGRAY_OK;
                                CK(cudaEventRecord(e1, stream));
                                CK(cudaStreamSynchronize(stream));
                                float ms = 0.f;
                                CK(cudaEventElapsedTime(&ms, e0, e1));
                                sh.times[r] = ms * 1000.0 / iters;
                            }
                            int bad = ok ? 0 : 1;
                            if (o.check && ok) {
                                // which output elements exist on this rank, and what they must hold
                                size_t out_len = len;
                                if (func == "all_gather" || func == "all_to_all") out_len = len * n;
                                if (func == "gather") out_len = r == static_cast<int>(root) ? len * n : 0;
                                if (func == "reduce" && r != static_cast<int>(root)) out_len = 0;
                                if (func == "send_recv") out_len = r == 1 ? len : 0;
                                const size_t P = kPatternBytes / dt.size;
                                auto expected = [&](size_t i) -> double {
                                    auto red = [&](size_t at) {
                                        double acc = sh.pattern[0][at % P];
                                        for (int q = 1; q < n; ++q) {
                                            const double v = sh.pattern[q][at % P];
                                            acc = op == MEGRAY_SUM ? acc + v : op == MEGRAY_MAX ? std::max(acc, v) : std::min(acc, v);
                                        }
                                        return acc;
                                    };
                                    if (func == "all_reduce" || func == "reduce") return red(i);
                                    if (func == "reduce_scatter") return red(r * len + i);
                                    if (func == "all_gather" || func == "gather") return sh.pattern[i / len][(i % len) % P];
                                    if (func == "all_to_all") return sh.pattern[i / len][(r * len + i % len) % P];
                                    if (func == "broadcast") return sh.pattern[root][i % P];
                                    if (func == "scatter") return sh.pattern[root][(r * len + i) % P];
                                    return sh.pattern[0][i % P];  // send_recv
                                };
                                // three windows of the output: its start, its middle and its end
                                const size_t win = std::min<size_t>(out_len, 8192);
                                const size_t starts[3] = {0, out_len > win ? (out_len - win) / 2 : 0, out_len - win};
                                const double tol = is_reducing(func) ? tolerance(dt, n) : 0.0;
                                for (int w = 0; w < 3 && win > 0; ++w) {
                                    window.resize(win * dt.size);
                                    if (host)
                                        memcpy(window.data(), out + starts[w] * dt.size, win * dt.size);
                                    else
                                        CK(cudaMemcpy(window.data(), out + starts[w] * dt.size, win * dt.size,
                                                      cudaMemcpyDeviceToHost));
                                    for (size_t i = 0; i < win; ++i) {
                                        double want = expected(starts[w] + i);
                                        if (dt.kind == K_INT || dt.kind == K_UINT) {
                                            // integer sums wrap like the element type
                                            const double span = ldexp(1.0, static_cast<int>(8 * dt.size));
                                            if (dt.size < 8) {
                                                want = fmod(want, span);
                                                if (dt.kind == K_INT && want >= span / 2) want -= span;
                                                if (dt.kind == K_INT && want < -span / 2) want += span;
                                                if (dt.kind == K_UINT && want < 0) want += span;
                                            }
                                        }
                                        const double got = read_value(dt, window.data() + i * dt.size);
                                        if (!(fabs(got - want) <= tol * std::max(1.0, fabs(want)))) ++bad;
                                    }
                                }
                            }
                            sh.bad[r] = bad;
                            sh.bar.wait();
                            if (r == 0) {
                                const double t_us = *std::max_element(sh.times.begin(), sh.times.end());
                                int total_bad = 0;
                                for (int b : sh.bad) total_bad += b;
                                const double speed = size / t_us / 1000.0;
                                const double busbw = speed * bus_factor(func, n);
                                const char* algo = "-";
#ifndef MEGRAY_BENCH_REFERENCE
                                const CommStats st1 = comm->stats();
                                if (st1.algo_nvls > st0.algo_nvls) algo = "nvls";
                                else if (st1.algo_ll > st0.algo_ll) algo = "flagged-words";
                                else if (st1.algo_direct > st0.algo_direct) algo = "single-pass";
                                else if (st1.algo_oneshot > st0.algo_oneshot) algo = "one-shot";
                                else if (st1.algo_twoshot > st0.algo_twoshot) algo = "staged";
                                else if (st1.algo_copy > st0.algo_copy) algo = "staged-copy";
                                else if (backend == MEGRAY_NCCL) algo = "nccl";
#endif
                                std::string phases;
#ifndef MEGRAY_BENCH_REFERENCE
                                if (o.phases && backend == MEGRAY_NVL) {
                                    // rank 0's last kernel: microseconds between its phase boundaries
                                    uint64_t st[8];
                                    const int ns = as_nvl(comm.get())->read_phase_stamps(st, 8);
                                    for (int i = 1; i < ns; ++i) {
                                        char buf[32];
                                        snprintf(buf, sizeof(buf), "%s%.2f", i > 1 ? "," : "", (st[i] - st[i - 1]) / 1000.0);
                                        phases += buf;
                                    }
                                }
#endif
                                if (o.json)
                                    printf("{\"backend\":\"%s\",\"op\":\"%s\",\"dtype\":\"%s\",\"reduce\":\"%s\",\"nranks\":%d,"
                                           "\"bytes\":%zu,\"time_us\":%.3f,\"speed_gbs\":%.3f,\"busbw_gbs\":%.3f,\"algo\":\"%s\","
                                           "\"phases_us\":[%s],\"checked\":%s,\"ok\":%s}\n",
                                           bname.c_str(), func.c_str(), dt.name, opname.c_str(), n, size, t_us, speed, busbw,
                                           algo, phases.c_str(), o.check ? "true" : "false", total_bad == 0 ? "true" : "false");
                                else
                                    printf("%-14s %-8s %-4s %12zu %12.2f %12.3f %12.3f  %-13s%s%s%s\n", func.c_str(), dt.name,
                                           opname.c_str(), size, t_us, speed, busbw, algo, phases.empty() ? "" : "  phases(us) ",
                                           phases.c_str(), total_bad == 0 ? "" : "  FAILED");
                                fflush(stdout);
                            }
                            sh.bar.wait();
                        }
                    }
                }
            }
#ifndef MEGRAY_BENCH_REFERENCE
            if (registered) {
                NvlInterface* nvl = as_nvl(comm.get());
                nvl->deregister_buffer(out);
                nvl->deregister_buffer(in);
            }
#endif
            comm.reset();
            if (host) {
                free(in);
                free(out);
            } else {
                cudaEventDestroy(e0);
                cudaEventDestroy(e1);
                if (!from_heap) {
                    cudaFree(in);
                    cudaFree(out);
                }
                cudaStreamDestroy(stream);
            }
        });
    }
    for (auto& t : threads) t.join();
}

void usage() {
    printf("megray_bench [-d devices] [-e nccl,nvl] [-f all_reduce,...|all] [-s 1K:1G | 8,1024,...]\n"
           "             [-t dtype,...|all] [-o sum,max,min|all] [-w warmup] [-i iters] [-j] [-c (check results)]\n"
           "             [-H (NVL: symmetric-heap buffers)] [-R (NVL: register the cudaMalloc buffers)]\n"
           "             [-C (shm backend with CPU ranks: host buffers, wall-clock timing; automatic without GPUs)]\n"
           "             [-p (NVL: time between the phase boundaries of rank 0's last kernel of each case)]\n"
           "             [-I master_ip] [-P port] [-n nodes] [-r node_rank]\n");
}

}  // namespace

int main(int argc, char** argv) {
    BenchOptions o;
    std::string sizes = "8,1K,512K,1M,10M";  // the reference tool's defaults (test/performance.cpp:59)
    std::string backends = "nccl";
    std::string funcs = "all";
    std::string dtypes = "float32", ops = "sum";
    int c;
    while ((c = getopt(argc, argv, "d:I:P:n:r:e:f:s:w:i:t:o:jcHRCph")) != -1) {
        switch (c) {
            case 'd': o.devices = atoi(optarg); break;
            case 'I': o.master_ip = optarg; break;
            case 'P': o.port = atoi(optarg); break;
            case 'n': o.nodes = atoi(optarg); break;
            case 'r': o.node_rank = atoi(optarg); break;
            case 'e': backends = optarg; break;
            case 'f': funcs = optarg; break;
            case 's': sizes = optarg; break;
            case 'w': o.warmup = atoi(optarg); break;
            case 'i': o.iters = atoi(optarg); break;
            case 't': dtypes = optarg; break;
            case 'o': ops = optarg; break;
            case 'j': o.json = true; break;
            case 'c': o.check = true; break;
            case 'H': o.heap = true; break;
            case 'R': o.reg = true; break;
            case 'C': o.host = true; break;
            case 'p': o.phases = true; setenv("MEGRAY_PHASES", "1", 1); break;
            default: usage(); return c == 'h' ? 0 : 1;
        }
    }
    if (o.nodes != 1) {
        fprintf(stderr, "megray_bench drives the GPUs of one node (-n 1); start one copy per node by hand "
                        "as with the reference tool if a multi-node NCCL run is wanted\n");
        return 1;
    }
    o.backends = split(backends, ',');
    if (funcs == "all")
        for (const char* f : kAllFuncs) o.funcs.push_back(f);
    else
        o.funcs = split(funcs, ',');
    if (sizes.find(':') != std::string::npos) {
        auto lr = split(sizes, ':');
        for (size_t s = parse_size(lr[0]); s <= parse_size(lr[1]); s *= 2) o.sizes.push_back(s);
    } else {
        for (auto& s : split(sizes, ',')) o.sizes.push_back(parse_size(s));
    }
    if (dtypes == "all")
        for (const auto& d : kDTypes) o.dtypes.push_back(d.name);
    else
        o.dtypes = split(dtypes, ',');
    for (const auto& name : o.dtypes) {
        bool known = false;
        for (const auto& d : kDTypes) known = known || name == d.name;
        if (!known) {
            fprintf(stderr, "unknown dtype %s\n", name.c_str());
            return 1;
        }
    }
    o.ops = ops == "all" ? std::vector<std::string>{"sum", "max", "min"} : split(ops, ',');
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess) {
        (void)cudaGetLastError();
        ndev = 0;
    }
    bool only_shm = true;
    for (const auto& b : o.backends) only_shm = only_shm && b == "shm";
    if (ndev < o.devices && only_shm) o.host = true;  // CPU ranks: the timed CPU baseline
    if (!o.host && ndev < o.devices) {
        fprintf(stderr, "%d devices wanted, %d present (the shm backend alone also runs with CPU ranks: -C)\n",
                o.devices, ndev);
        return 1;
    }
    setenv("NCCL_LAUNCH_MODE", "PARALLEL", 0);  // the reference's NCCL backend insists on it

    for (const auto& bname : o.backends) {
        if (!o.json) {
            printf("\n%s, %d devices\n", bname.c_str(), o.devices);
            printf("%-14s %-8s %-4s %12s %12s %12s %12s  %s\n", "function", "dtype", "op", "bufsize", "time(us)",
                   "speed(GB/s)", "busbw(GB/s)", "algorithm");
        }
        const int port = o.port > 0 ? o.port : get_free_port();
        if (create_server(static_cast<uint32_t>(o.devices), port) != MEGRAY_OK) {
            fprintf(stderr, "cannot start the rendezvous server on port %d\n", port);
            return 1;
        }
        run_backend(o, bname, backend_of(bname), port);
    }
    return 0;
}
