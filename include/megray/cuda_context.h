/**
 * CUDA stream context (reference include/megray/cuda_context.h:46-57): device
 * buffers; operations are enqueued on the wrapped stream and return at once.
 */
#pragma once
#include <memory>

#include "megray/context.h"

#ifdef MEGRAY_WITH_CUDA
#include <cuda_runtime_api.h>

namespace MegRay {

class CudaContext : public Context {
public:
    CudaContext() : m_stream(nullptr) {}
    explicit CudaContext(cudaStream_t stream) : m_stream(stream) {}
    static std::shared_ptr<CudaContext> make(cudaStream_t stream) {
        return std::make_shared<CudaContext>(stream);
    }
    ContextType type() const override { return MEGRAY_CTX_CUDA; }
    cudaStream_t get_stream() { return m_stream; }

private:
    cudaStream_t m_stream;
};

}  // namespace MegRay
#endif  // MEGRAY_WITH_CUDA
