/**
 * Execution contexts: where an operation is ordered.
 *
 * The reference declares MEGRAY_CTX_DEFAULT but ships no class for it
 * (include/megray/context.h:19-35).  Here `HostContext` is that class: buffers
 * are host memory and calls complete before they return (host backend).
 */
#pragma once
#include <memory>

#include "megray/common.h"

namespace MegRay {

typedef enum {
    MEGRAY_CTX_DEFAULT = 0,
    MEGRAY_CTX_CUDA = 1,
    MEGRAY_CTX_HIP = 2,
    MEGRAY_CTX_COUNT = 3,
} ContextType;

class Context {
public:
    virtual ContextType type() const = 0;
    virtual ~Context() = default;
};

/** Host buffers, synchronous completion. */
class HostContext : public Context {
public:
    HostContext() = default;
    static std::shared_ptr<HostContext> make() { return std::make_shared<HostContext>(); }
    ContextType type() const override { return MEGRAY_CTX_DEFAULT; }
};

}  // namespace MegRay
