// C++ test binary over the public interface, ranks as threads of one process.
//
// Re-expresses the reference's gtest suite (reference test/test_server_client.cpp,
// test/test_opr.cpp, test/test_shm.cpp) for this library: rendezvous calls, communicator
// init for every built backend, and the ten operations with the reference's closed-form
// inputs (float32, 10 elements, value (i+1)*(j+1), 3 ranks, root 1).  The host backend
// cases run anywhere; the NCCL / NVL cases need one GPU per rank and are skipped otherwise.
//
//   megray_test [filter]        run the tests whose name contains `filter`
#include <cuda_runtime.h>
#include <math.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "host/shared_region.h"
#include "megray.h"
#include "mini_test.h"

using namespace MegRay;

namespace {

int gpu_count() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

void run_ranks(int n, const std::function<void(int)>& fn) {
    std::vector<std::thread> th;
    std::mutex mu;
    std::vector<std::string> errors;
    for (int r = 0; r < n; ++r)
        th.emplace_back([&, r] {
            try {
                fn(r);
            } catch (const std::exception& e) {
                std::lock_guard<std::mutex> lk(mu);
                errors.push_back("rank " + std::to_string(r) + ": " + e.what());
            }
        });
    for (auto& t : th) t.join();
    for (auto& e : errors) {
        ++mini::failures();
        printf("  %s\n", e.c_str());
    }
}

// Device abstraction of the tests: host buffers for the host backend, device buffers +
// stream for the CUDA backends (the reference's ContextTrait, test/test_utils.h:19-75).
struct Env {
    bool cuda;
    cudaStream_t stream = nullptr;
    std::shared_ptr<Context> ctx;
    Env(bool use_cuda, int rank) : cuda(use_cuda) {
        if (cuda) {
            cudaSetDevice(rank);
            cudaStreamCreate(&stream);
            ctx = CudaContext::make(stream);
        } else {
            ctx = HostContext::make();
        }
    }
    ~Env() {
        if (cuda && stream) cudaStreamDestroy(stream);
    }
    void* alloc(size_t bytes) {
        void* p = nullptr;
        if (cuda) cudaMalloc(&p, bytes);
        else p = malloc(bytes);
        return p;
    }
    void release(void* p) {
        if (cuda) cudaFree(p);
        else free(p);
    }
    void put(void* dst, const void* src, size_t bytes) {
        if (cuda) cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice);
        else memcpy(dst, src, bytes);
    }
    void get(void* dst, const void* src, size_t bytes) {
        if (cuda) {
            cudaStreamSynchronize(stream);
            cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost);
        } else {
            memcpy(dst, src, bytes);
        }
    }
};

struct BackendCase {
    Backend backend;
    const char* name;
    bool cuda;
};
std::vector<BackendCase> backends(int nranks) {
    std::vector<BackendCase> b = {{MEGRAY_SHM, "shm", false}};
    if (gpu_count() >= nranks) {
        b.push_back({MEGRAY_NVL, "nvl", true});
        b.push_back({MEGRAY_NCCL, "nccl", true});
    }
    return b;
}

// run `body(comm, env, rank)` for every available backend
void for_all_backends(int nranks,
                      const std::function<void(Communicator&, Env&, int, const BackendCase&)>& body) {
    for (const auto& bc : backends(nranks)) {
        Server server(static_cast<uint32_t>(nranks));
        const int port = server.port();
        run_ranks(nranks, [&](int rank) {
            Env env(bc.cuda, rank);
            auto comm = get_communicator(nranks, rank, bc.backend);
            if (comm->init("127.0.0.1", port) != MEGRAY_OK)
                throw std::runtime_error(std::string("init failed on ") + bc.name);
            body(*comm, env, rank, bc);
        });
    }
}

float cf(int i, int j) { return static_cast<float>((i + 1) * (j + 1)); }

}  // namespace

// ------------------------------------------------------------------ rendezvous

TEST(ServerClient_GetHostIp) {
    char* ip = get_host_ip();
    if (ip != nullptr) {
        EXPECT_TRUE(strlen(ip) >= 7);
        delete[] ip;
    }
}

TEST(ServerClient_GetFreePort) { EXPECT_TRUE(get_free_port() > 0); }

TEST(ServerClient_Connect) {
    const int n = 3;
    const int port = get_free_port();
    EXPECT_EQ(create_server(n, port), MEGRAY_OK);
    run_ranks(n, [&](int r) {
        Client c(n, r);
        ASSERT_TRUE(c.connect("127.0.0.1", port) == MEGRAY_OK);
    });
}

TEST(ServerClient_Barrier) {
    const int n = 3;
    Server server(n);
    std::atomic<int> counter{0};
    run_ranks(n, [&](int r) {
        Client c(n, r);
        ASSERT_TRUE(c.connect("127.0.0.1", server.port()) == MEGRAY_OK);
        usleep(50000 * r);
        ++counter;
        ASSERT_TRUE(c.barrier() == MEGRAY_OK);
        EXPECT_EQ(counter.load(), n);
    });
}

TEST(ServerClient_Broadcast) {
    const int n = 3, root = 1;
    Server server(n);
    const char* msg = "0123456789abcdefghij";
    run_ranks(n, [&](int r) {
        Client c(n, r);
        ASSERT_TRUE(c.connect("127.0.0.1", server.port()) == MEGRAY_OK);
        char out[10] = {0};
        ASSERT_TRUE(c.broadcast(msg + r * 5, out, 10, root) == MEGRAY_OK);
        EXPECT_TRUE(memcmp(out, msg + root * 5, 10) == 0);
    });
}

TEST(ServerClient_AllGather) {
    const int n = 3;
    Server server(n);
    run_ranks(n, [&](int r) {
        Client c(n, r);
        ASSERT_TRUE(c.connect("127.0.0.1", server.port()) == MEGRAY_OK);
        char mine[4] = {static_cast<char>('a' + r), static_cast<char>('A' + r), 0, 1};
        char all[12];
        ASSERT_TRUE(c.allgather(mine, all, 4) == MEGRAY_OK);
        for (int q = 0; q < n; ++q) {
            EXPECT_EQ(all[4 * q], 'a' + q);
            EXPECT_EQ(all[4 * q + 1], 'A' + q);
        }
    });
}

TEST(ServerClient_Sequence) {
    const int n = 3;
    Server server(n);
    run_ranks(n, [&](int r) {
        Client c(n, r);
        ASSERT_TRUE(c.connect("127.0.0.1", server.port()) == MEGRAY_OK);
        int v = r == 2 ? 42 : 0, got = 0;
        ASSERT_TRUE(c.barrier() == MEGRAY_OK);
        ASSERT_TRUE(c.broadcast(&v, &got, sizeof(int), 2) == MEGRAY_OK);
        EXPECT_EQ(got, 42);
        int all[3];
        ASSERT_TRUE(c.allgather(&r, all, sizeof(int)) == MEGRAY_OK);
        EXPECT_TRUE(all[0] == 0 && all[1] == 1 && all[2] == 2);
        ASSERT_TRUE(c.barrier() == MEGRAY_OK);
    });
    EXPECT_EQ(server.requests_served(), 4u);
}

// ------------------------------------------------------------------ communicators

TEST(Communicator_InitEveryBackend) {
    int seen = 0;
    for_all_backends(3, [&](Communicator& comm, Env&, int rank, const BackendCase& bc) {
        EXPECT_EQ(comm.nranks(), 3u);
        EXPECT_EQ(comm.rank(), static_cast<uint32_t>(rank));
        EXPECT_EQ(comm.backend(), bc.backend);
        if (rank == 0) ++seen;
    });
    EXPECT_TRUE(seen >= 1);
}

// init(BcastCallback): no rendezvous server at all; the caller supplies the broadcast (here a
// board in this process), as the reference's embedding framework does
// (include/megray/communicator.h:46-47 of the reference).
TEST(Communicator_InitWithBroadcastCallback) {
    const int n = 3;
    struct Board {
        std::mutex mu;
        std::condition_variable cv;
        std::vector<char> data;
        int generation = 0;  // messages published so far
        int taken = 0;       // readers that have copied the current message
    } board;
    run_ranks(n, [&](int rank) {
        int seen = 0;  // messages this rank has been through
        auto bcast = [&board, &seen, rank, n](char* buf, size_t len) {
            std::unique_lock<std::mutex> lk(board.mu);
            if (rank == 0) {
                board.cv.wait(lk, [&] { return board.generation == 0 || board.taken == n - 1; });
                board.data.assign(buf, buf + len);
                board.taken = 0;
                ++board.generation;
            } else {
                board.cv.wait(lk, [&] { return board.generation > seen; });
                memcpy(buf, board.data.data(), len);
                ++board.taken;
            }
            ++seen;
            board.cv.notify_all();
        };
        auto comm = get_communicator(n, rank, MEGRAY_SHM);
        if (comm->init(bcast) != MEGRAY_OK) throw std::runtime_error("init(callback) failed");
        std::vector<float> in(10), out(10, 0.f);
        for (int j = 0; j < 10; ++j) in[j] = cf(rank, j);
        if (comm->all_reduce(in.data(), out.data(), 10, MEGRAY_FLOAT32, MEGRAY_SUM, HostContext::make()) != MEGRAY_OK)
            throw std::runtime_error("all_reduce failed");
        for (int j = 0; j < 10; ++j)
            if (out[j] != cf(0, j) + cf(1, j) + cf(2, j)) throw std::runtime_error("wrong sum");
    });
}

TEST(Communicator_UnknownBackendsThrow) {
    for (Backend b : {MEGRAY_UCX, MEGRAY_RCCL}) {
        bool threw = false;
        try {
            get_communicator(2, 0, b);
        } catch (const Exception&) {
            threw = true;
        }
        EXPECT_TRUE(threw);
    }
}

TEST(Opr_SendRecv) {
    const char* msg = "test_message";
    const size_t len = strlen(msg);
    for_all_backends(2, [&](Communicator& comm, Env& env, int rank, const BackendCase&) {
        void* buf = env.alloc(len);
        if (rank == 0) {
            env.put(buf, msg, len);
            ASSERT_TRUE(comm.send(buf, len, MEGRAY_CHAR, 1, env.ctx) == MEGRAY_OK);
            char tmp[16];
            env.get(tmp, buf, len);  // synchronises the stream before the buffer goes away
        } else {
            ASSERT_TRUE(comm.recv(buf, len, MEGRAY_CHAR, 0, env.ctx) == MEGRAY_OK);
            char out[16] = {0};
            env.get(out, buf, len);
            EXPECT_TRUE(memcmp(out, msg, len) == 0);
        }
        env.release(buf);
    });
}

TEST(Opr_ScatterGather) {
    const int n = 3, len = 10, root = 1;
    for_all_backends(n, [&](Communicator& comm, Env& env, int rank, const BackendCase&) {
        std::vector<float> full(n * len), part(len, 0.f), back(n * len, 0.f);
        for (int i = 0; i < n; ++i)
            for (int j = 0; j < len; ++j) full[i * len + j] = cf(i, j);
        void* d_full = rank == root ? env.alloc(n * len * 4) : nullptr;  // null on non-root ranks
        void* d_part = env.alloc(len * 4);
        void* d_back = rank == root ? env.alloc(n * len * 4) : nullptr;
        if (rank == root) env.put(d_full, full.data(), n * len * 4);
        ASSERT_TRUE(comm.scatter(d_full, d_part, len, MEGRAY_FLOAT32, root, env.ctx) == MEGRAY_OK);
        env.get(part.data(), d_part, len * 4);
        for (int j = 0; j < len; ++j) EXPECT_EQ(part[j], cf(rank, j));
        ASSERT_TRUE(comm.gather(d_part, d_back, len, MEGRAY_FLOAT32, root, env.ctx) == MEGRAY_OK);
        if (rank == root) {
            env.get(back.data(), d_back, n * len * 4);
            for (int k = 0; k < n * len; ++k) EXPECT_EQ(back[k], full[k]);
            env.release(d_full);
            env.release(d_back);
        } else {
            float tmp;
            env.get(&tmp, d_part, 4);
        }
        env.release(d_part);
    });
}

TEST(Opr_AllToAll) {
    const int n = 3, len = 2;
    for_all_backends(n, [&](Communicator& comm, Env& env, int rank, const BackendCase&) {
        std::vector<float> in(n * len), out(n * len, -1.f);
        for (int q = 0; q < n; ++q)
            for (int j = 0; j < len; ++j) in[q * len + j] = static_cast<float>(100 * rank + 10 * q + j);
        void* d_in = env.alloc(n * len * 4);
        void* d_out = env.alloc(n * len * 4);
        env.put(d_in, in.data(), n * len * 4);
        ASSERT_TRUE(comm.all_to_all(d_in, d_out, len, MEGRAY_FLOAT32, env.ctx) == MEGRAY_OK);
        env.get(out.data(), d_out, n * len * 4);
        for (int q = 0; q < n; ++q)
            for (int j = 0; j < len; ++j) EXPECT_EQ(out[q * len + j], static_cast<float>(100 * q + 10 * rank + j));
        env.release(d_in);
        env.release(d_out);
    });
}

TEST(Opr_AllGather) {
    const int n = 3, len = 10;
    for_all_backends(n, [&](Communicator& comm, Env& env, int rank, const BackendCase&) {
        std::vector<float> in(len), out(n * len, 0.f);
        for (int j = 0; j < len; ++j) in[j] = cf(rank, j);
        void* d_in = env.alloc(len * 4);
        void* d_out = env.alloc(n * len * 4);
        env.put(d_in, in.data(), len * 4);
        ASSERT_TRUE(comm.all_gather(d_in, d_out, len, MEGRAY_FLOAT32, env.ctx) == MEGRAY_OK);
        env.get(out.data(), d_out, n * len * 4);
        for (int i = 0; i < n; ++i)
            for (int j = 0; j < len; ++j) EXPECT_EQ(out[i * len + j], cf(i, j));
        env.release(d_in);
        env.release(d_out);
    });
}

static float expect_reduce(int n, int j, ReduceOp op) {
    float acc = cf(0, j);
    for (int i = 1; i < n; ++i) {
        const float v = cf(i, j);
        acc = op == MEGRAY_SUM ? acc + v : op == MEGRAY_MAX ? fmaxf(acc, v) : fminf(acc, v);
    }
    return acc;
}

TEST(Opr_AllReduce_ReduceScatter_Reduce) {
    const int n = 3, len = 10, root = 1;
    for (ReduceOp op : {MEGRAY_SUM, MEGRAY_MAX, MEGRAY_MIN}) {
        for_all_backends(n, [&](Communicator& comm, Env& env, int rank, const BackendCase&) {
            const int total = n * len;
            std::vector<float> in(total), ar(total, 0.f), rs(len, 0.f), rd(total, 0.f);
            for (int j = 0; j < total; ++j) in[j] = cf(rank, j);
            void* d_in = env.alloc(total * 4);
            void* d_ar = env.alloc(total * 4);
            void* d_rs = env.alloc(len * 4);
            void* d_rd = env.alloc(total * 4);  // left uninitialised on non-root ranks
            env.put(d_in, in.data(), total * 4);
            ASSERT_TRUE(comm.all_reduce(d_in, d_ar, total, MEGRAY_FLOAT32, op, env.ctx) == MEGRAY_OK);
            ASSERT_TRUE(comm.reduce_scatter(d_in, d_rs, len, MEGRAY_FLOAT32, op, env.ctx) == MEGRAY_OK);
            ASSERT_TRUE(comm.reduce(d_in, d_rd, total, MEGRAY_FLOAT32, op, root, env.ctx) == MEGRAY_OK);
            env.get(ar.data(), d_ar, total * 4);
            env.get(rs.data(), d_rs, len * 4);
            env.get(rd.data(), d_rd, total * 4);
            for (int j = 0; j < total; ++j) EXPECT_EQ(ar[j], expect_reduce(n, j, op));
            for (int j = 0; j < len; ++j) EXPECT_EQ(rs[j], expect_reduce(n, rank * len + j, op));
            if (rank == root)
                for (int j = 0; j < total; ++j) EXPECT_EQ(rd[j], expect_reduce(n, j, op));
            env.release(d_in);
            env.release(d_ar);
            env.release(d_rs);
            env.release(d_rd);
        });
    }
}

TEST(Opr_Broadcast) {
    const int n = 3, len = 10, root = 1;
    for_all_backends(n, [&](Communicator& comm, Env& env, int rank, const BackendCase&) {
        std::vector<float> in(len), out(len, 0.f);
        for (int j = 0; j < len; ++j) in[j] = cf(rank, j);
        void* d_in = env.alloc(len * 4);
        void* d_out = env.alloc(len * 4);
        env.put(d_in, in.data(), len * 4);
        ASSERT_TRUE(comm.broadcast(d_in, d_out, len, MEGRAY_FLOAT32, root, env.ctx) == MEGRAY_OK);
        env.get(out.data(), d_out, len * 4);
        for (int j = 0; j < len; ++j) EXPECT_EQ(out[j], cf(root, j));  // on the root too
        env.release(d_in);
        env.release(d_out);
    });
}

TEST(Opr_ReduceRejectsChar) {
    for_all_backends(2, [&](Communicator& comm, Env& env, int, const BackendCase&) {
        void* b = env.alloc(16);
        EXPECT_EQ(comm.all_reduce(b, b, 16, MEGRAY_CHAR, MEGRAY_SUM, env.ctx), MEGRAY_INVALID_ARGUMENT);
        env.release(b);
    });
}

TEST(Nvl_SymmetricAllocAndScaledAllReduce) {
    const int n = std::min(gpu_count(), 4);
    if (n < 2) SKIP("needs two GPUs");
    Server server(n);
    run_ranks(n, [&](int rank) {
        Env env(true, rank);
        auto comm = get_communicator(n, rank, MEGRAY_NVL);
        ASSERT_TRUE(comm->init("127.0.0.1", server.port()) == MEGRAY_OK);
        NvlInterface* nvl = as_nvl(comm.get());
        ASSERT_TRUE(nvl != nullptr);
        size_t off = 0;
        void* a = nvl->sym_alloc(4096, &off);
        ASSERT_TRUE(a != nullptr && nvl->in_heap(a, 4096));
        ASSERT_TRUE(nvl->peer_ptr(a, (rank + 1) % n) != nullptr);
        const int len = 1000;
        std::vector<float> in(len, static_cast<float>(rank + 1)), out(len, 0.f);
        void* d_in = env.alloc(len * 4);
        void* d_out = env.alloc(len * 4);
        env.put(d_in, in.data(), len * 4);
        ASSERT_TRUE(nvl->all_reduce_scaled(d_in, d_out, len, MEGRAY_FLOAT32, MEGRAY_FLOAT32, 1.0f / n, MEGRAY_SUM,
                                           env.ctx) == MEGRAY_OK);
        env.get(out.data(), d_out, len * 4);
        for (int j = 0; j < len; ++j) EXPECT_TRUE(fabsf(out[j] - (n + 1) / 2.0f) < 1e-5f);
        EXPECT_EQ(nvl->sym_free(a), MEGRAY_OK);
        env.release(d_in);
        env.release(d_out);
    });
}

// ------------------------------------------------------------------ shared region of the host backend
// (the counterpart of the reference's test/test_shm.cpp: shared memory write / read, and the
// synchronisation built in it, from one thread and from two)
TEST(Shm_RegionWriteReadInProcess) {
    const std::string name = "megray-test-region-" + std::to_string(getpid()) + "-a";
    auto owner = host::SharedRegion::create(name, 2, 4096, 1024, true);
    ASSERT_TRUE(owner != nullptr);
    auto peer = host::SharedRegion::attach(name, true, 1000);
    ASSERT_TRUE(peer != nullptr);
    EXPECT_EQ(peer->nranks(), 2u);
    EXPECT_EQ(peer->slot_bytes(), owner->slot_bytes());
    for (int i = 0; i < 4096; ++i) owner->slot(1)[i] = static_cast<char>(i * 7);
    int wrong = 0;
    for (int i = 0; i < 4096; ++i) wrong += peer->slot(1)[i] != static_cast<char>(i * 7);
    EXPECT_EQ(wrong, 0);
    // one mailbox per ordered pair, distinct storage
    EXPECT_TRUE(owner->mailbox_data(0, 1) != owner->mailbox_data(1, 0));
    peer->mailbox_data(0, 1)[5] = 42;
    EXPECT_EQ(owner->mailbox_data(0, 1)[5], 42);
}

TEST(Shm_RegionWriteReadPosixObject) {
    const std::string name = "megray-test-region-" + std::to_string(getpid()) + "-b";
    auto owner = host::SharedRegion::create(name, 3, 1 << 16, 4096, false);
    ASSERT_TRUE(owner != nullptr);
    auto peer = host::SharedRegion::attach(name, false, 1000);  // a second mapping of the object
    ASSERT_TRUE(peer != nullptr);
    EXPECT_TRUE(static_cast<void*>(peer->slot(0)) != static_cast<void*>(owner->slot(0)));
    memset(owner->result(), 0x5a, 1 << 16);
    int wrong = 0;
    for (int i = 0; i < (1 << 16); ++i) wrong += peer->result()[i] != 0x5a;
    EXPECT_EQ(wrong, 0);
    EXPECT_TRUE(host::SharedRegion::attach(name + "-absent", false, 50) == nullptr);
}

TEST(Shm_BarrierTwoThreads) {
    const std::string name = "megray-test-region-" + std::to_string(getpid()) + "-c";
    auto region = host::SharedRegion::create(name, 2, 256, 256, true);
    ASSERT_TRUE(region != nullptr);
    std::atomic<int> arrived{0};
    std::atomic<int> ahead{0};
    const int rounds = 2000;
    run_ranks(2, [&](int rank) {
        auto mine = rank == 0 ? region : host::SharedRegion::attach(name, true, 1000);
        uint32_t sense = 0;
        for (int i = 0; i < rounds; ++i) {
            arrived.fetch_add(1);
            if (mine->barrier(&sense, 5000) != MEGRAY_OK) throw std::runtime_error("barrier failed");
            // nobody leaves round i before both ranks have arrived in it
            if (arrived.load() < 2 * (i + 1)) ahead.fetch_add(1);
        }
    });
    EXPECT_EQ(ahead.load(), 0);
    EXPECT_EQ(arrived.load(), 2 * rounds);
}

TEST(Shm_BarrierTimeoutAndAbort) {
    const std::string name = "megray-test-region-" + std::to_string(getpid()) + "-d";
    auto region = host::SharedRegion::create(name, 2, 256, 256, true);
    ASSERT_TRUE(region != nullptr);
    uint32_t sense = 0;
    EXPECT_EQ(region->barrier(&sense, 50), MEGRAY_TIMEOUT);  // the second rank never comes
    region->abort();
    EXPECT_TRUE(region->aborted());
    uint32_t sense2 = 0;
    EXPECT_EQ(region->barrier(&sense2, 50), MEGRAY_ABORTED);
}

// A message many times the size of the ring mailbox crosses it in pieces, in both directions
// at once (the reference's RingSender / RingRecver pair, test/test_shm.cpp:57-83).
TEST(Shm_MailboxCarriesMessagesLargerThanTheRing) {
    setenv("MEGRAY_HOST_MAILBOX_KB", "4", 1);
    Server server(2);
    const size_t len = 1 << 20;
    run_ranks(2, [&](int rank) {
        auto comm = get_communicator(2, rank, MEGRAY_SHM);
        if (comm->init("127.0.0.1", server.port()) != MEGRAY_OK) throw std::runtime_error("init");
        auto ctx = HostContext::make();
        std::vector<char> out(len), in(len, 0);
        for (size_t i = 0; i < len; ++i) out[i] = static_cast<char>((i * 31 + rank) & 0xff);
        if (comm->group_start() != MEGRAY_OK) throw std::runtime_error("group_start");
        comm->send(out.data(), len, MEGRAY_CHAR, 1 - rank, ctx);
        comm->recv(in.data(), len, MEGRAY_CHAR, 1 - rank, ctx);
        if (comm->group_end() != MEGRAY_OK) throw std::runtime_error("group_end");
        size_t wrong = 0;
        for (size_t i = 0; i < len; ++i) wrong += in[i] != static_cast<char>((i * 31 + (1 - rank)) & 0xff);
        if (wrong) throw std::runtime_error("payload differs");
    });
    unsetenv("MEGRAY_HOST_MAILBOX_KB");
}

// Ranks as threads of one process: a registered cudaMalloc buffer is reached by its plain
// address once peer access is enabled (no IPC handle involved).
TEST(Nvl_RegisteredUserBuffersTakeTheSinglePassKernels) {
    const int n = std::min(gpu_count(), 4);
    if (n < 2) SKIP("needs two GPUs");
    Server server(n);
    run_ranks(n, [&](int rank) {
        Env env(true, rank);
        auto comm = get_communicator(n, rank, MEGRAY_NVL);
        ASSERT_TRUE(comm->init("127.0.0.1", server.port()) == MEGRAY_OK);
        NvlInterface* nvl = as_nvl(comm.get());
        ASSERT_TRUE(nvl != nullptr);
        const size_t len = (1u << 20) + 8;  // above the one-shot limit
        std::vector<float> in(len), out(len, 0.f);
        for (size_t j = 0; j < len; ++j) in[j] = static_cast<float>((rank + 1) * (1 + j % 7));
        void* d_in = env.alloc(len * 4);
        void* d_out = env.alloc(len * 4);
        void* d_gather = env.alloc(len * 4 * n);
        env.put(d_in, in.data(), len * 4);
        ASSERT_TRUE(nvl->register_buffer(d_in, len * 4) == MEGRAY_OK);
        ASSERT_TRUE(nvl->register_buffer(d_out, len * 4) == MEGRAY_OK);
        ASSERT_TRUE(nvl->register_buffer(d_gather, len * 4 * n) == MEGRAY_OK);
        const CommStats before = comm->stats();
        ASSERT_TRUE(comm->all_reduce(d_in, d_out, len, MEGRAY_FLOAT32, MEGRAY_SUM, env.ctx) == MEGRAY_OK);
        env.get(out.data(), d_out, len * 4);
        const float tri = n * (n + 1) / 2.0f;
        size_t wrong = 0;
        for (size_t j = 0; j < len; ++j) wrong += out[j] != tri * (1 + j % 7);
        EXPECT_EQ(wrong, 0u);
        ASSERT_TRUE(comm->all_gather(d_in, d_gather, len, MEGRAY_FLOAT32, env.ctx) == MEGRAY_OK);
        std::vector<float> all(len * n);
        env.get(all.data(), d_gather, len * 4 * n);
        wrong = 0;
        for (int q = 0; q < n; ++q)
            for (size_t j = 0; j < len; j += 997) wrong += all[q * len + j] != static_cast<float>((q + 1) * (1 + j % 7));
        EXPECT_EQ(wrong, 0u);
        EXPECT_TRUE(comm->stats().calls >= before.calls + 2);
        EXPECT_EQ(nvl->deregister_buffer(d_gather), MEGRAY_OK);
        EXPECT_EQ(nvl->deregister_buffer(d_out), MEGRAY_OK);
        EXPECT_EQ(nvl->deregister_buffer(d_in), MEGRAY_OK);
        EXPECT_TRUE(nvl->deregister_buffer(d_in) != MEGRAY_OK);
        env.release(d_in);
        env.release(d_out);
        env.release(d_gather);
    });
}

int main(int argc, char** argv) {
    setenv("NCCL_LAUNCH_MODE", "PARALLEL", 0);
    return mini::run_all(argc > 1 ? argv[1] : nullptr);
}
