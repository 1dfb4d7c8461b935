// A second, independent model of the reducing collectives: instead of combining the ranks'
// inputs in rank order (cpu_reduce_n), it replays the step-by-step schedules of the reference's
// host-driven backend over host buffers: the ring all_reduce (reduce-scatter ring followed by an
// all-gather ring, src/ucx/all_reduce.cpp:61-101 of the reference) and the binomial-tree reduce
// (src/ucx/reduce.cpp:42-80).  Every pairwise combination is rounded to the element type, as a
// per-step kernel would.  Integer and MAX / MIN results must equal the rank-order oracle bit for
// bit; floating-point sums may differ by the reassociation only, which bounds what any schedule
// of the device kernels may legitimately produce.
#pragma once
#include <stddef.h>

#include "megray/types.h"

namespace MegRay {
namespace host {

/** Ring all_reduce of `nranks` inputs of `len` elements; `out[r]` receives rank r's result. */
Status ring_all_reduce_schedule(const void* const* in, void* const* out, int nranks, size_t len,
                                DType dtype, ReduceOp op);

/** Binomial-tree reduce towards `root`; `out` receives the root's result. */
Status tree_reduce_schedule(const void* const* in, void* out, int nranks, int root, size_t len,
                            DType dtype, ReduceOp op);

}  // namespace host
}  // namespace MegRay
