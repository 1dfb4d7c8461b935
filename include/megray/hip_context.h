/**
 * HIP stream context, kept only for source compatibility with code that
 * includes it under MEGRAY_WITH_HIP (reference include/megray/hip_context.h).
 * No backend of this library consumes it: B200 is a CUDA platform.
 */
#pragma once
#include "megray/context.h"

#ifdef MEGRAY_WITH_HIP
#include <hip/hip_runtime.h>

namespace MegRay {
class HipContext : public Context {
public:
    explicit HipContext(hipStream_t stream) : m_stream(stream) {}
    static std::shared_ptr<HipContext> make(hipStream_t stream) {
        return std::make_shared<HipContext>(stream);
    }
    ContextType type() const override { return MEGRAY_CTX_HIP; }
    hipStream_t get_stream() { return m_stream; }

private:
    hipStream_t m_stream;
};
}  // namespace MegRay
#endif
