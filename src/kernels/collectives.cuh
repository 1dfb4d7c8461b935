// Launch interface of the native collective kernels (sm_100a, NVLink peer memory).
//
// Two kernel families serve all ten MegRay operations:
//
//   reduce family  (all_reduce, reduce_scatter, reduce, fused scale/cast all_reduce)
//     phase P  push   : rank r stores slice j of its input into peer j's staging slot [r]
//                       (the copy-in is the NVLink transfer; user buffers need no registration)
//     barrier
//     phase R  reduce : rank r combines its n staging slots in rank order (fp32 accumulation
//                       for fp16/bf16), applies scale and the output cast, and keeps the
//                       reduced slice in its `red` buffer (and in its own output)
//     barrier
//     phase G  gather : ranks that want the full result load the reduced slices from the
//                       peers' `red` buffers straight into their output
//     One-shot variant (small messages): every rank pushes its whole input to every peer,
//     one barrier, local reduce.
//
//   exchange family (all_gather, all_to_all, broadcast, gather, scatter)
//     phase P  publish: copy the chunks others will read into the local `pub` buffer, or
//                       (bandwidth-optimal broadcast) the root pushes slice j to peer j
//     barrier
//     phase G  gather : each rank loads what it needs from the peers' `pub` buffers into
//                       its output
//
// Work is partitioned so that CTA c of one rank only ever depends on CTA c of the other
// ranks; barriers are per CTA: one flag word per (CTA, peer) in each rank's signal pad,
// written with st.release.sys and polled with ld.acquire.sys against a monotonically
// increasing epoch.  Every wait is bounded; when one runs out the kernel records
// MEGRAY_TIMEOUT in the status word, skips its remaining phases and returns.
//
// The reference reaches the same operations through ncclAllReduce & co.
// (reference src/nccl/communicator.cpp:162-228) or host-driven ring steps with a
// one-element-per-thread reduce kernel (reference src/ucx/kernel.cu:16-60).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "megray/types.h"

namespace mgk {
namespace coll {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 128;        // flag rows in a signal pad
constexpr int kPadBytes = 64 * 1024; // signal pad at the start of every rank's heap

struct PeerTable {
    // peer q's heap base address as mapped in this rank's address space
    char* heap[kMaxRanks];
};

struct CommonArgs {
    PeerTable peers;
    int nranks;
    int rank;
    uint32_t epoch;        // first barrier of this launch waits for epoch+1
    uint64_t timeout_ns;   // limit of one wait
    int* status;           // device-visible status word (0 = ok)
    uint64_t flag_off;     // byte offset of the flag rows inside the heap
};

struct ReduceArgs {
    CommonArgs c;
    const void* in;        // user input (len_total elements of in_dtype)
    void* out;             // user output, may be null on ranks that do not gather
    uint64_t slice_elems;  // elements per slice (the last slice may be shorter)
    uint64_t len;          // total elements covered by this launch (<= nranks * slice_elems)
    uint64_t stage_off;    // byte offset of the staging slots inside the heap
    uint64_t red_off;      // byte offset of the reduced-slice buffer inside the heap
    float scale;           // applied to SUM results of floating dtypes when != 1
    int one_shot;          // 1: push everything everywhere, single barrier
    int do_gather;         // phase G wanted on this rank
    int out_is_slice;      // reduce_scatter: out holds only this rank's slice
    uint64_t in_pitch_elems;  // slice j of the input starts at element j*in_pitch_elems
    MegRay::DType in_dtype;
    MegRay::DType out_dtype;
    MegRay::ReduceOp op;
};

struct ExchangeArgs {
    CommonArgs c;
    const void* in;
    void* out;
    uint64_t pub_off;       // byte offset of the publish buffer inside the heap
    uint64_t chunk_bytes;   // bytes of one chunk (piece) moved by this launch
    uint64_t in_pitch;      // bytes between consecutive chunks in `in`
    uint64_t out_pitch;     // bytes between consecutive chunks in `out`
    int publish_chunks;     // chunks this rank copies from `in` to its pub buffer (0 = none)
    int push_root;          // >= 0: two-step broadcast, that rank pushes slice j to peer j
    uint32_t pull_mask;     // bit q set: load a chunk from peer q
    // chunk loaded from peer q: pub[q] + src_chunk[q]*chunk_bytes  ->  out + dst_chunk[q]*chunk_bytes
    int src_chunk[kMaxRanks];
    int dst_chunk[kMaxRanks];
    uint64_t pull_bytes[kMaxRanks];  // bytes to load from peer q (<= chunk_bytes)
    // Small messages, push form: instead of publishing locally and loading from the peers
    // (a load's round trip after the barrier), chunk push_chunk[j] of `in` is stored into slot
    // `rank` of peer j's pub buffer before the barrier, and after it the n slots are copied
    // from the local pub buffer to `out` chunk q.  The stores' latency hides behind the flag's.
    int push_all;
    int push_chunk[kMaxRanks];
};

// Single-pass ("direct") collectives for buffers that live in the symmetric heap at the same
// offset on every rank: no staging at all.
//   all_reduce      barrier; rank r loads slice r of all n inputs straight from the peers' heaps
//                   (or, with NVLS, one multimem.ld_reduce that the NVSwitch reduces), combines,
//                   scales, casts and stores the result into all n outputs (one multimem.st with
//                   NVLS); barrier.  Loads and stores overlap, so both link directions are busy.
//   reduce_scatter  barrier; load slice r of all inputs, combine, store locally; barrier.
//   all_gather      barrier; store this rank's block into slot r of all n outputs; barrier.
//   all_to_all      barrier; store chunk q of this rank's input into slot r of rank q's output; barrier.
enum DirectKind : int {
    DIRECT_ALL_REDUCE = 0,
    DIRECT_REDUCE_SCATTER = 1,
    DIRECT_ALL_GATHER = 2,
    DIRECT_ALL_TO_ALL = 3
};

struct DirectArgs {
    CommonArgs c;
    int kind;
    // every rank's input (all_reduce, reduce_scatter) and output (all_reduce, all_gather,
    // all_to_all) buffer as mapped in this rank's address space: heap addresses, or peer mappings
    // of buffers registered with the communicator
    const char* in_base[kMaxRanks];
    char* out_base[kMaxRanks];
    uint64_t in_off;       // heap offset of the input: the multimem address is mc_base + in_off
    uint64_t out_off;      // heap offset of the output
    const void* in_local;  // all_gather / all_to_all: this rank's input (any device memory)
    void* out_local;       // reduce_scatter: this rank's result (any device memory)
    uint64_t len;          // all_reduce: total elements; others: elements per rank
    float scale;
    MegRay::DType in_dtype;
    MegRay::DType out_dtype;
    MegRay::ReduceOp op;
    char* mc_base;         // non-null: multicast (NVLS) mapping of the heap, use multimem
};

// True if the NVSwitch can reduce this dtype/op pair (multimem.ld_reduce): bf16/fp16 all ops,
// fp32 SUM; the rest takes peer loads.
bool nvls_supports(MegRay::DType in_dtype, MegRay::DType out_dtype, MegRay::ReduceOp op);

cudaError_t launch_direct(const DirectArgs& args, int ctas, int threads, cudaStream_t stream);

cudaError_t launch_reduce(const ReduceArgs& args, int ctas, int threads, cudaStream_t stream);
cudaError_t launch_exchange(const ExchangeArgs& args, int ctas, int threads, cudaStream_t stream);

// Stand-alone N-way elementwise reduction out = op(in[0..n)) on one GPU (the device
// counterpart of the reference's reduce kernels, src/ucx/kernel.cu:16-60), with the same
// fp32 accumulation, scale and cast as the collectives.
cudaError_t launch_reduce_n(const void* const* in, int n_in, void* out, uint64_t len,
                            MegRay::DType in_dtype, MegRay::DType out_dtype, MegRay::ReduceOp op,
                            float scale, cudaStream_t stream);

}  // namespace coll
}  // namespace mgk
