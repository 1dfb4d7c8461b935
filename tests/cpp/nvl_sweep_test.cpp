// All ten operations of the NVL backend against values computed on the host, ranks as threads
// of one process (the way the reference's tests drive their ranks, test/test_base.h:46-51), on
// plain cudaMalloc buffers: over element types, the three reductions, lengths that fall on
// every size class (flagged-word kernel, one-shot, single-pass kernels on the peers' buffers),
// ragged lengths, and buffers that start off the 16-byte grid.  With one GPU the same sweep runs
// on a single-rank group, which still launches the same kernels.
//
// Inputs are small integers in every element type, so every sum is exact and independent of
// the order of the additions: results must match bit for bit.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "megray.h"
#include "mini_test.h"

using namespace MegRay;

namespace {

int device_count() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

// value of element i on rank r (salt separates the buffers of different calls)
int value(int r, size_t i, int salt, bool is_unsigned) {
    const int v = static_cast<int>((i * 131u + static_cast<unsigned>(r) * 71u + static_cast<unsigned>(salt) * 29u) % 17u);
    return is_unsigned ? v : v - 8;
}

uint16_t to_half_bits(int v) {  // exact for |v| < 2048
    if (v == 0)
        return 0;
    const uint16_t sign = v < 0 ? 0x8000 : 0;
    unsigned a = static_cast<unsigned>(v < 0 ? -v : v);
    int e = 0;
    while ((a >> (e + 1)) != 0) ++e;             // a in [2^e, 2^(e+1))
    const unsigned mant = (a << (10 - e)) & 0x3ff;  // e <= 10
    return static_cast<uint16_t>(sign | ((e + 15) << 10) | mant);
}
long from_half_bits(uint16_t h) {
    if ((h & 0x7fff) == 0)
        return 0;
    const int e = ((h >> 10) & 0x1f) - 15;
    const unsigned long m = 0x400 | (h & 0x3ff);
    const long a = e >= 10 ? static_cast<long>(m << (e - 10)) : (e > -22 ? static_cast<long>(m >> (10 - e)) : 0);
    return (h & 0x8000) ? -a : a;
}
uint16_t to_bf16_bits(int v) {  // exact for |v| <= 256
    const float f = static_cast<float>(v);
    uint32_t u;
    memcpy(&u, &f, 4);
    return static_cast<uint16_t>(u >> 16);
}
long from_bf16_bits(uint16_t b) {
    const uint32_t u = static_cast<uint32_t>(b) << 16;
    float f;
    memcpy(&f, &u, 4);
    return static_cast<long>(f);
}

struct TypeCase {
    DType dtype;
    size_t size;
    bool is_unsigned;
    const char* name;
};
const TypeCase kTypes[] = {
        {MEGRAY_FLOAT32, 4, false, "float32"}, {MEGRAY_BFLOAT16, 2, false, "bfloat16"}, {MEGRAY_FLOAT16, 2, false, "float16"},
        {MEGRAY_INT32, 4, false, "int32"},     {MEGRAY_UINT32, 4, true, "uint32"},      {MEGRAY_INT8, 1, false, "int8"},
        {MEGRAY_UINT8, 1, true, "uint8"},      {MEGRAY_INT64, 8, false, "int64"},       {MEGRAY_UINT64, 8, true, "uint64"},
        {MEGRAY_FLOAT64, 8, false, "float64"},
};

void encode(const TypeCase& t, int v, char* dst) {
    switch (t.dtype) {
        case MEGRAY_FLOAT32: { float x = static_cast<float>(v); memcpy(dst, &x, 4); break; }
        case MEGRAY_FLOAT64: { double x = v; memcpy(dst, &x, 8); break; }
        case MEGRAY_FLOAT16: { uint16_t x = to_half_bits(v); memcpy(dst, &x, 2); break; }
        case MEGRAY_BFLOAT16: { uint16_t x = to_bf16_bits(v); memcpy(dst, &x, 2); break; }
        case MEGRAY_INT32: case MEGRAY_UINT32: { int32_t x = v; memcpy(dst, &x, 4); break; }
        case MEGRAY_INT64: case MEGRAY_UINT64: { int64_t x = v; memcpy(dst, &x, 8); break; }
        default: { int8_t x = static_cast<int8_t>(v); memcpy(dst, &x, 1); }
    }
}
long decode(const TypeCase& t, const char* src) {
    switch (t.dtype) {
        case MEGRAY_FLOAT32: { float x; memcpy(&x, src, 4); return static_cast<long>(x); }
        case MEGRAY_FLOAT64: { double x; memcpy(&x, src, 8); return static_cast<long>(x); }
        case MEGRAY_FLOAT16: { uint16_t x; memcpy(&x, src, 2); return from_half_bits(x); }
        case MEGRAY_BFLOAT16: { uint16_t x; memcpy(&x, src, 2); return from_bf16_bits(x); }
        case MEGRAY_INT32: { int32_t x; memcpy(&x, src, 4); return x; }
        case MEGRAY_UINT32: { uint32_t x; memcpy(&x, src, 4); return static_cast<long>(x); }
        case MEGRAY_INT64: case MEGRAY_UINT64: { int64_t x; memcpy(&x, src, 8); return static_cast<long>(x); }
        case MEGRAY_UINT8: { uint8_t x; memcpy(&x, src, 1); return x; }
        default: { int8_t x; memcpy(&x, src, 1); return x; }
    }
}

long reduce_expected(int n, size_t i, int salt, bool uns, ReduceOp op) {
    long acc = value(0, i, salt, uns);
    for (int r = 1; r < n; ++r) {
        const long v = value(r, i, salt, uns);
        acc = op == MEGRAY_SUM ? acc + v : op == MEGRAY_MAX ? (v > acc ? v : acc) : (v < acc ? v : acc);
    }
    return acc;
}

struct Failures {
    std::mutex mu;
    std::vector<std::string> what;
    void add(const std::string& s) {
        std::lock_guard<std::mutex> lk(mu);
        if (what.size() < 20)
            what.push_back(s);
    }
};

// One rank's part of the sweep.  `skew`: bytes by which every buffer starts off the 256-byte
// grid of cudaMalloc (0, or one element).
void sweep_rank(int n, int rank, int port, const std::vector<size_t>& lens, size_t max_len, Failures& fails) {
    cudaSetDevice(rank);
    cudaStream_t stream;
    cudaStreamCreate(&stream);
    auto ctx = CudaContext::make(stream);
    auto comm = get_communicator(n, rank, MEGRAY_NVL);
    if (comm->init("127.0.0.1", port) != MEGRAY_OK)
        throw std::runtime_error("init failed");
    const size_t cap = max_len * 8 * n + 64;
    char *d_in = nullptr, *d_out = nullptr;
    cudaMalloc(&d_in, cap);
    cudaMalloc(&d_out, cap);
    std::vector<char> h_in(cap), h_out(cap);
    const int root = 1 % n;
    int salt = 0;
    for (const TypeCase& t : kTypes) {
        for (size_t len : lens) {
            if (t.size < 4 && t.dtype != MEGRAY_BFLOAT16 && len > 100000)
                continue;  // the long lengths with the main element types only
            if (t.size == 8 && len > 100000 && t.dtype != MEGRAY_FLOAT64)
                continue;
            for (int skewed = 0; skewed < 2; ++skewed) {
                if (skewed && len > 100000 && t.dtype != MEGRAY_FLOAT32)
                    continue;
                const size_t skew = skewed ? t.size : 0;
                char* in = d_in + skew;
                char* out = d_out + skew;
                ++salt;
                // input: n * len elements (the widest any operation reads)
                const size_t in_elems = len * n;
                for (size_t i = 0; i < in_elems; ++i) encode(t, value(rank, i, salt, t.is_unsigned), &h_in[i * t.size]);
                cudaMemcpyAsync(in, h_in.data(), in_elems * t.size, cudaMemcpyHostToDevice, stream);
                auto fetch = [&](size_t elems) {
                    cudaMemcpyAsync(h_out.data(), out, elems * t.size, cudaMemcpyDeviceToHost, stream);
                    cudaStreamSynchronize(stream);
                };
                auto clear = [&](size_t elems) { cudaMemsetAsync(out, 0x5a, elems * t.size, stream); };
                auto tag = [&](const char* op) {
                    return std::string(op) + " " + t.name + " len " + std::to_string(len) + (skewed ? " skewed" : "") +
                           " rank " + std::to_string(rank) + "/" + std::to_string(n);
                };
                auto expect = [&](const char* op, size_t elems, const std::function<long(size_t)>& want) {
                    size_t bad = 0, first = 0;
                    for (size_t i = 0; i < elems; ++i) {
                        if (decode(t, &h_out[i * t.size]) != want(i)) {
                            if (bad == 0)
                                first = i;
                            ++bad;
                        }
                    }
                    if (bad)
                        fails.add(tag(op) + ": " + std::to_string(bad) + " wrong, first at " + std::to_string(first) +
                                  " got " + std::to_string(decode(t, &h_out[first * t.size])) + " want " +
                                  std::to_string(want(first)));
                };
                const bool uns = t.is_unsigned;
                for (ReduceOp op : {MEGRAY_SUM, MEGRAY_MAX, MEGRAY_MIN}) {
                    if (op != MEGRAY_SUM && len > 100000)
                        continue;
                    clear(len);
                    if (comm->all_reduce(in, out, len, t.dtype, op, ctx) != MEGRAY_OK) fails.add(tag("all_reduce call"));
                    fetch(len);
                    expect("all_reduce", len, [&](size_t i) { return reduce_expected(n, i, salt, uns, op); });
                    clear(len);
                    if (comm->reduce_scatter(in, out, len, t.dtype, op, ctx) != MEGRAY_OK) fails.add(tag("reduce_scatter call"));
                    fetch(len);
                    expect("reduce_scatter", len, [&](size_t i) { return reduce_expected(n, rank * len + i, salt, uns, op); });
                    clear(len);
                    if (comm->reduce(in, rank == root ? out : nullptr, len, t.dtype, op, root, ctx) != MEGRAY_OK)
                        fails.add(tag("reduce call"));
                    fetch(len);
                    if (rank == root)
                        expect("reduce", len, [&](size_t i) { return reduce_expected(n, i, salt, uns, op); });
                    else
                        expect("reduce (untouched)", len, [&](size_t) { return decode(t, "\x5a\x5a\x5a\x5a\x5a\x5a\x5a\x5a"); });
                }
                clear(len * n);
                if (comm->all_gather(in, out, len, t.dtype, ctx) != MEGRAY_OK) fails.add(tag("all_gather call"));
                fetch(len * n);
                expect("all_gather", len * n, [&](size_t i) { return static_cast<long>(value(static_cast<int>(i / len), i % len, salt, uns)); });
                clear(len * n);
                if (comm->all_to_all(in, out, len, t.dtype, ctx) != MEGRAY_OK) fails.add(tag("all_to_all call"));
                fetch(len * n);
                expect("all_to_all", len * n,
                       [&](size_t i) { return static_cast<long>(value(static_cast<int>(i / len), rank * len + i % len, salt, uns)); });
                clear(len);
                if (comm->broadcast(rank == root ? in : nullptr, out, len, t.dtype, root, ctx) != MEGRAY_OK)
                    fails.add(tag("broadcast call"));
                fetch(len);
                expect("broadcast", len, [&](size_t i) { return static_cast<long>(value(root, i, salt, uns)); });
                clear(len * n);
                if (comm->gather(in, rank == root ? out : nullptr, len, t.dtype, root, ctx) != MEGRAY_OK)
                    fails.add(tag("gather call"));
                fetch(len * n);
                if (rank == root)
                    expect("gather", len * n, [&](size_t i) { return static_cast<long>(value(static_cast<int>(i / len), i % len, salt, uns)); });
                clear(len);
                if (comm->scatter(rank == root ? in : nullptr, out, len, t.dtype, root, ctx) != MEGRAY_OK)
                    fails.add(tag("scatter call"));
                fetch(len);
                expect("scatter", len, [&](size_t i) { return static_cast<long>(value(root, rank * len + i, salt, uns)); });
            }
        }
    }
    cudaStreamSynchronize(stream);
    if (comm->status() != MEGRAY_OK)
        fails.add("communicator status " + std::to_string(comm->status()) + " on rank " + std::to_string(rank));
    const CommStats st = comm->stats();
    NvlInterface* nvl = as_nvl(comm.get());
    if (nvl == nullptr || nvl->check_canaries() != MEGRAY_OK)
        fails.add("a guard zone around the staging workspaces was overwritten on rank " + std::to_string(rank));
    if (st.algo_ll == 0 || st.algo_direct == 0)
        fails.add("expected both the flagged-word and the single-pass kernels to run: ll " + std::to_string(st.algo_ll) +
                  " direct " + std::to_string(st.algo_direct));
    comm.reset();
    cudaFree(d_in);
    cudaFree(d_out);
    cudaStreamDestroy(stream);
}

void run_sweep(int n) {
    // elements per rank unit: flagged words (<= 16-32 KiB), their ragged tails, the one-shot
    // all_reduce range, and the single-pass kernels (ragged and not)
    const std::vector<size_t> lens = {1, 5, 1000, 4099, 9000, 70001, 300007, (1u << 20) + 3};
    Server server(static_cast<uint32_t>(n));
    Failures fails;
    std::vector<std::thread> th;
    std::mutex mu;
    for (int r = 0; r < n; ++r)
        th.emplace_back([&, r] {
            try {
                sweep_rank(n, r, server.port(), lens, lens.back(), fails);
            } catch (const std::exception& e) {
                fails.add(std::string("rank ") + std::to_string(r) + ": " + e.what());
            }
        });
    for (auto& t : th) t.join();
    for (const auto& f : fails.what) {
        ++mini::failures();
        printf("  %s\n", f.c_str());
    }
}

}  // namespace

TEST(Nvl_SingleRankGroupRunsEveryOperation) {
    if (device_count() < 1) SKIP("needs a GPU");
    run_sweep(1);
}

TEST(Nvl_AllOperationsOnPlainBuffersAgainstHostValues) {
    const int n = std::min(device_count(), 8);
    if (n < 2) SKIP("needs two GPUs");
    run_sweep(n);
    // Once more with few CTAs, small chunks and the staged forms of reduce from 100 KB on: the
    // pipelined broadcast and the staged reduces then run many chunks per CTA, more than a CTA has
    // staging slots, so slots are reused under the consumed-chunk counters.  Form 1: the root
    // pushes its input; form 2: the root loads the reduced chunks (run together with the
    // broadcast in which every rank loads instead of the root and the slice owners storing).
    setenv("MEGRAY_REDUCE_STAGED_MIN", "100000", 1);
    setenv("MEGRAY_BCAST_CHUNK", "16384", 1);
    setenv("MEGRAY_DIRECT_CTA_BYTES", "262144", 1);
    setenv("MEGRAY_REDUCE_MODE", "1", 1);
    run_sweep(n);
    setenv("MEGRAY_REDUCE_MODE", "2", 1);
    setenv("MEGRAY_BCAST_PULL", "1", 1);  // and the broadcast by loads alone
    run_sweep(n);
    if (n > 3)
        run_sweep(3);  // an odd group: slices and chunk shares that do not divide evenly
    setenv("MEGRAY_REDUCE_MODE", "3", 1);  // form 3: in steps separated by barriers, loads only
    setenv("MEGRAY_REDUCE_STEPS", "3", 1);
    run_sweep(n > 3 ? 3 : n);
    if (n > 3)
        run_sweep(n);
    unsetenv("MEGRAY_REDUCE_STEPS");
    unsetenv("MEGRAY_REDUCE_STAGED_MIN");
    unsetenv("MEGRAY_BCAST_CHUNK");
    unsetenv("MEGRAY_DIRECT_CTA_BYTES");
    unsetenv("MEGRAY_REDUCE_MODE");
    unsetenv("MEGRAY_BCAST_PULL");
    if (n > 3)
        run_sweep(3);
}

// The range guard of a build with MEGRAY_DEBUG_BOUNDS, exercised without any access that is really
// out of bounds: with MEGRAY_DEBUG_BOUNDS_SELFTEST=1 the communicator tells its kernels that the
// call's buffers are half as long as they are, so the guard must refuse the ranges that reach into
// the second half (skipping them), record the first one and report MEGRAY_OUT_OF_BOUNDS.  Runs
// only when the environment says that this binary is such a build.
TEST(Nvl_RangeGuardRefusesWhatLiesOutsideTheDeclaredBuffers) {
    if (getenv("MEGRAY_EXPECT_BOUNDS_BUILD") == nullptr || getenv("MEGRAY_DEBUG_BOUNDS_SELFTEST") == nullptr)
        SKIP("needs the bounds-checked build and its self-test mode");
    if (device_count() < 1) SKIP("needs a GPU");
    for (size_t len : {size_t(1000), size_t(1) << 20}) {  // flagged-word kernel, single-pass kernel
        Server server(1);
        cudaSetDevice(0);
        cudaStream_t stream;
        cudaStreamCreate(&stream);
        auto ctx = CudaContext::make(stream);
        auto comm = get_communicator(1, 0, MEGRAY_NVL);
        ASSERT_TRUE(comm->init("127.0.0.1", server.port()) == MEGRAY_OK);
        float *in = nullptr, *out = nullptr;
        cudaMalloc(&in, len * 4);
        cudaMalloc(&out, len * 4);
        std::vector<float> h(len, 3.0f);
        cudaMemcpy(in, h.data(), len * 4, cudaMemcpyHostToDevice);
        cudaMemset(out, 0, len * 4);
        EXPECT_EQ(comm->all_reduce(in, out, len, MEGRAY_FLOAT32, MEGRAY_SUM, ctx), MEGRAY_OK);
        cudaStreamSynchronize(stream);
        EXPECT_EQ(comm->status(), MEGRAY_OUT_OF_BOUNDS);
        cudaMemcpy(h.data(), out, len * 4, cudaMemcpyDeviceToHost);
        EXPECT_EQ(h[len - 1], 0.0f);  // the refused range was not written
        // the context is intact and a later call is refused with the recorded status
        EXPECT_EQ(comm->all_reduce(in, out, len, MEGRAY_FLOAT32, MEGRAY_SUM, ctx), MEGRAY_OUT_OF_BOUNDS);
        EXPECT_EQ(cudaDeviceSynchronize(), cudaSuccess);
        comm.reset();
        cudaFree(in);
        cudaFree(out);
        cudaStreamDestroy(stream);
    }
}
