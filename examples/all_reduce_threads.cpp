// Smallest complete program on the C++ interface: N ranks as threads of one process meet through
// the TCP rendezvous and sum a vector.
//
//   all_reduce_threads [nranks] [backend: shm | nvl | nccl]
//
// `shm` (the default) needs no GPU: buffers are host memory and the context is a HostContext.
// `nvl` / `nccl` use GPU r for rank r and a CUDA stream per rank.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <thread>
#include <vector>

#include "megray.h"

int main(int argc, char** argv) {
    const int nranks = argc > 1 ? atoi(argv[1]) : 2;
    const char* name = argc > 2 ? argv[2] : "shm";
    const MegRay::Backend backend = !strcmp(name, "nvl")    ? MegRay::MEGRAY_NVL
                                    : !strcmp(name, "nccl") ? MegRay::MEGRAY_NCCL
                                                            : MegRay::MEGRAY_SHM;
    const bool cuda = backend != MegRay::MEGRAY_SHM;
    const size_t len = 1 << 20;

    MegRay::Server server(nranks);  // picks a free port, serves until it goes out of scope
    std::vector<int> bad(nranks, 0);
    std::vector<std::thread> ranks;
    for (int r = 0; r < nranks; ++r) {
        ranks.emplace_back([&, r] {
            std::vector<float> in(len, static_cast<float>(r + 1)), out(len, 0.f);
            auto comm = MegRay::get_communicator(nranks, r, backend);
            if (cuda)
                cudaSetDevice(r);
            if (comm->init("127.0.0.1", server.port()) != MegRay::MEGRAY_OK) {
                bad[r] = 1;
                return;
            }
            MegRay::Status st;
            if (!cuda) {
                st = comm->all_reduce(in.data(), out.data(), len, MegRay::MEGRAY_FLOAT32, MegRay::MEGRAY_SUM,
                                      MegRay::HostContext::make());
            } else {
                cudaStream_t stream;
                cudaStreamCreate(&stream);
                float *d_in, *d_out;
                cudaMalloc(&d_in, len * sizeof(float));
                cudaMalloc(&d_out, len * sizeof(float));
                cudaMemcpyAsync(d_in, in.data(), len * sizeof(float), cudaMemcpyHostToDevice, stream);
                st = comm->all_reduce(d_in, d_out, len, MegRay::MEGRAY_FLOAT32, MegRay::MEGRAY_SUM,
                                      MegRay::CudaContext::make(stream));
                cudaMemcpyAsync(out.data(), d_out, len * sizeof(float), cudaMemcpyDeviceToHost, stream);
                cudaStreamSynchronize(stream);
                cudaFree(d_in);
                cudaFree(d_out);
                cudaStreamDestroy(stream);
            }
            const float want = nranks * (nranks + 1) / 2.0f;
            if (st != MegRay::MEGRAY_OK)
                bad[r] = 1;
            for (size_t i = 0; i < len; ++i)
                if (out[i] != want)
                    bad[r] = 1;
        });
    }
    for (auto& t : ranks)
        t.join();
    int failed = 0;
    for (int b : bad)
        failed += b;
    printf("%s all_reduce of %zu floats over %d ranks: %s\n", name, len, nranks, failed ? "FAILED" : "ok");
    return failed ? 1 : 0;
}
