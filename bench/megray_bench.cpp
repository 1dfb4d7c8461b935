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
//   * any dtype (-t) and reduce op (-o), sizes given in bytes or as a doubling range
//     (-s 1K:1G), JSON lines with -j, buffers filled with seeded data and (with -c)
//     results checked against the host oracle.
// Ranks are threads of this process, one GPU each (as the reference's tests and benchmark
// drive them).  Because it uses only the interface shared with the reference, this file
// also compiles against the reference's own headers and objects (-DMEGRAY_BENCH_REFERENCE):
// that build is the like-for-like baseline.
#include <cuda_runtime.h>

#include <chrono>
#include <getopt.h>
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
    std::string dtype = "float32";
    std::string op = "sum";
    bool json = false;
    bool check = false;
    bool heap = false;  // NVL backend: buffers from the symmetric heap (zero-copy / NVSwitch kernels)
    bool reg = false;   // NVL backend: cudaMalloc buffers registered with the communicator (zero-copy)
    bool host = false;  // shm backend with CPU ranks: host buffers, wall-clock timing, no GPU needed
};

const char* kAllFuncs[] = {"send_recv", "scatter", "gather", "all_to_all", "all_gather",
                           "all_reduce", "reduce_scatter", "broadcast", "reduce"};

struct DTypeInfo {
    const char* name;
    DType dtype;
    size_t size;
};
const DTypeInfo kDTypes[] = {
        {"int8", MEGRAY_INT8, 1},       {"uint8", MEGRAY_UINT8, 1},     {"int32", MEGRAY_INT32, 4},
        {"uint32", MEGRAY_UINT32, 4},   {"int64", MEGRAY_INT64, 8},     {"uint64", MEGRAY_UINT64, 8},
        {"float16", MEGRAY_FLOAT16, 2}, {"float32", MEGRAY_FLOAT32, 4}, {"float64", MEGRAY_FLOAT64, 8},
#ifndef MEGRAY_BENCH_REFERENCE
        {"bfloat16", MEGRAY_BFLOAT16, 2},
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

struct Result {
    double time_us;  // max over ranks, per call
    bool ok;
};

double bus_factor(const std::string& f, int n) {
    if (f == "all_reduce") return 2.0 * (n - 1) / n;
    if (f == "all_gather" || f == "reduce_scatter" || f == "all_to_all" || f == "gather" || f == "scatter")
        return static_cast<double>(n - 1);
    return 1.0;
}

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

// `unit` is the reference tool's notion of buffer size for the function (per-rank send size
// for all_gather, per-rank receive size for reduce_scatter, per-peer chunk for all_to_all /
// gather / scatter, the whole buffer otherwise: reference test/performance.cpp:153-252).
// One communicator group serves all sizes of a (backend, function) pair.
std::vector<Result> run_sizes(const BenchOptions& o, const std::string& func, Backend backend,
                              const std::vector<size_t>& sizes, const DTypeInfo& dt, ReduceOp op, int port) {
    const int n = o.devices;
    std::vector<std::vector<double>> times(sizes.size(), std::vector<double>(n, 0.0));
    std::vector<std::atomic<int>> bad(sizes.size());
    for (auto& b : bad) b = 0;
    std::atomic<bool> init_ok{true};
    ThreadBarrier bar(n);
    std::vector<std::thread> threads;
    size_t max_unit = 0;
    for (size_t s : sizes) max_unit = std::max(max_unit, s);
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
                init_ok = false;
            }
            if (comm && comm->init(o.master_ip.c_str(), port) != MEGRAY_OK) init_ok = false;
            bar.wait();
            if (!init_ok.load()) return;
            const size_t max_len = std::max<size_t>(1, max_unit / dt.size);
            const bool wide_in = func == "reduce_scatter" || func == "scatter" || func == "all_to_all";
            const bool wide_out = func == "all_gather" || func == "gather" || func == "all_to_all";
            void *in = nullptr, *out = nullptr;
            bool from_heap = false;
#ifndef MEGRAY_BENCH_REFERENCE
            if (o.heap && backend == MEGRAY_NVL) {
                NvlInterface* nvl = as_nvl(comm.get());
                in = nvl->sym_alloc(max_len * dt.size * (wide_in ? n : 1), nullptr);
                out = nvl->sym_alloc(max_len * dt.size * (wide_out ? n : 1), nullptr);
                from_heap = true;
                if (in == nullptr || out == nullptr) {
                    fprintf(stderr, "symmetric heap too small for these sizes: raise MEGRAY_HEAP_MB\n");
                    exit(1);
                }
            }
#endif
            if (host) {
                in = malloc(max_len * dt.size * (wide_in ? n : 1));
                out = malloc(max_len * dt.size * (wide_out ? n : 1));
            } else if (!from_heap) {
                CK(cudaMalloc(&in, max_len * dt.size * (wide_in ? n : 1)));
                CK(cudaMalloc(&out, max_len * dt.size * (wide_out ? n : 1)));
            }
#ifndef MEGRAY_BENCH_REFERENCE
            bool registered = false;
            if (!from_heap && o.reg && backend == MEGRAY_NVL) {
                NvlInterface* nvl = as_nvl(comm.get());
                const Status s1 = nvl->register_buffer(in, max_len * dt.size * (wide_in ? n : 1));
                const Status s2 = nvl->register_buffer(out, max_len * dt.size * (wide_out ? n : 1));
                registered = s1 == MEGRAY_OK && s2 == MEGRAY_OK;
                if (!registered && r == 0)
                    fprintf(stderr, "buffers could not be registered: staged paths\n");
            }
#endif
            cudaEvent_t e0 = nullptr, e1 = nullptr;
            if (host) {
                memset(in, r + 1, max_len * dt.size * (wide_in ? n : 1));
                memset(out, 0, max_len * dt.size * (wide_out ? n : 1));
            } else {
                CK(cudaMemset(in, r + 1, max_len * dt.size * (wide_in ? n : 1)));
                CK(cudaMemset(out, 0, max_len * dt.size * (wide_out ? n : 1)));
                CK(cudaEventCreate(&e0));
                CK(cudaEventCreate(&e1));
            }
            const uint32_t root = 0;
            for (size_t si = 0; si < sizes.size(); ++si) {
                const size_t len = std::max<size_t>(1, sizes[si] / dt.size);
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
                const int iters = sizes[si] >= (256u << 20) ? std::max(3, o.iters / 10) : o.iters;
                const int warm = sizes[si] >= (256u << 20) ? std::max(2, o.warmup / 10) : o.warmup;
                bool ok = true;
                for (int i = 0; i < warm && ok; ++i) ok = call() == MEGRAY_OK;
                if (host) {
                    // CPU ranks: the calls are synchronous, wall clock between two thread barriers
                    bar.wait();
                    const auto t0 = std::chrono::steady_clock::now();
                    for (int i = 0; i < iters && ok; ++i) ok = call() == MEGRAY_OK;
                    const auto t1 = std::chrono::steady_clock::now();
                    times[si][r] = std::chrono::duration<double, std::micro>(t1 - t0).count() / iters;
                } else {
                    CK(cudaStreamSynchronize(stream));
                    bar.wait();
                    CK(cudaEventRecord(e0, stream));
                    for (int i = 0; i < iters && ok; ++i) ok = call() == MEGRAY_OK;
                    CK(cudaEventRecord(e1, stream));
                    CK(cudaStreamSynchronize(stream));
                    float ms = 0.f;
                    CK(cudaEventElapsedTime(&ms, e0, e1));
                    times[si][r] = ms * 1000.0 / iters;
                }
                if (!ok) bad[si]++;
                if (o.check && ok && func == "all_reduce" && op == MEGRAY_SUM && dt.dtype == MEGRAY_UINT8) {
                    // every input byte is rank+1: the sum is n(n+1)/2 modulo 256
                    std::vector<uint8_t> h(std::min<size_t>(len, 4096));
                    if (host)
                        memcpy(h.data(), out, h.size());
                    else
                        CK(cudaMemcpy(h.data(), out, h.size(), cudaMemcpyDeviceToHost));
                    const uint8_t want = static_cast<uint8_t>(n * (n + 1) / 2);
                    for (uint8_t v : h)
                        if (v != want) bad[si]++;
                }
                bar.wait();
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
    std::vector<Result> res(sizes.size());
    for (size_t si = 0; si < sizes.size(); ++si) {
        res[si].time_us = *std::max_element(times[si].begin(), times[si].end());
        res[si].ok = init_ok.load() && bad[si].load() == 0;
    }
    return res;
}

void usage() {
    printf("megray_bench [-d devices] [-e nccl,nvl] [-f all_reduce,...|all] [-s 1K:1G | 8,1024,...]\n"
           "             [-t dtype] [-o sum|max|min] [-w warmup] [-i iters] [-j] [-c] [-H (NVL: symmetric-heap buffers)]\n"
           "             [-R (NVL: register the cudaMalloc buffers with the communicator)]\n"
           "             [-C (shm backend with CPU ranks: host buffers, wall-clock timing; automatic without GPUs)]\n"
           "             [-I master_ip] [-P port] [-n nodes] [-r node_rank]\n");
}

}  // namespace

int main(int argc, char** argv) {
    BenchOptions o;
    std::string sizes = "8,1K,512K,1M,10M";  // the reference tool's defaults (test/performance.cpp:59)
    std::string backends = "nccl";
    std::string funcs = "all";
    int c;
    while ((c = getopt(argc, argv, "d:I:P:n:r:e:f:s:w:i:t:o:jcHRCh")) != -1) {
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
            case 't': o.dtype = optarg; break;
            case 'o': o.op = optarg; break;
            case 'j': o.json = true; break;
            case 'c': o.check = true; break;
            case 'H': o.heap = true; break;
            case 'R': o.reg = true; break;
            case 'C': o.host = true; break;
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
    const DTypeInfo* dt = nullptr;
    for (const auto& d : kDTypes)
        if (o.dtype == d.name) dt = &d;
    if (dt == nullptr) {
        fprintf(stderr, "unknown dtype %s\n", o.dtype.c_str());
        return 1;
    }
    ReduceOp op = o.op == "max" ? MEGRAY_MAX : o.op == "min" ? MEGRAY_MIN : MEGRAY_SUM;
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
        for (const auto& func : o.funcs) {
            if (!o.json) {
                printf("\n%s / %s / %s / %s, %d devices\n", bname.c_str(), func.c_str(), dt->name, o.op.c_str(),
                       o.devices);
                printf("%14s %12s %14s %14s %8s\n", "bufsize", "time(us)", "speed(GB/s)", "busbw(GB/s)", "iters");
            }
            const int port = o.port > 0 ? o.port : get_free_port();
            if (create_server(static_cast<uint32_t>(o.devices), port) != MEGRAY_OK) {
                fprintf(stderr, "cannot start the rendezvous server on port %d\n", port);
                return 1;
            }
            std::vector<Result> results = run_sizes(o, func, backend_of(bname), o.sizes, *dt, op, port);
            for (size_t si = 0; si < o.sizes.size(); ++si) {
                const size_t bytes = o.sizes[si];
                const Result& r = results[si];
                const double speed = bytes / r.time_us / 1000.0;
                const double busbw = speed * bus_factor(func, o.devices);
                if (o.json)
                    printf("{\"backend\":\"%s\",\"op\":\"%s\",\"dtype\":\"%s\",\"reduce\":\"%s\",\"nranks\":%d,"
                           "\"bytes\":%zu,\"time_us\":%.3f,\"speed_gbs\":%.3f,\"busbw_gbs\":%.3f,\"ok\":%s}\n",
                           bname.c_str(), func.c_str(), dt->name, o.op.c_str(), o.devices, bytes, r.time_us, speed,
                           busbw, r.ok ? "true" : "false");
                else
                    printf("%14zu %12.2f %14.3f %14.3f %8d%s\n", bytes, r.time_us, speed, busbw, o.iters,
                           r.ok ? "" : "  FAILED");
                fflush(stdout);
            }
        }
    }
    return 0;
}
