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

// Layout of the first 16 KiB of the pad (byte offsets from the start of a rank's heap):
constexpr uint64_t kBarrierFlagOff = 0;      // [kMaxCtas][kMaxRanks] u32: per-CTA barrier epochs
constexpr uint64_t kChunkFlagOff = 4096;     // [kMaxCtas] u32: chunk counters of the pipelined broadcast
constexpr uint64_t kExchangeOff = 8192;      // [2][kMaxRanks] x 16 bytes: the buffers of the current call
constexpr uint64_t kTokenOff = 8192 + 512;   // [2][kMaxRanks] x 8 bytes: tokens of the small-message kernel
constexpr uint64_t kDebugOff = 8192 + 1024;  // bounds-checked build: the first access it refused
                                             // {u64 address, u64 bytes, u32 source line, u32 rank}
constexpr uint64_t kPhaseOff = 8192 + 2048;  // kMaxPhases x u64: %globaltimer stamps of CTA 0 (phase mode)
constexpr int kMaxPhases = 8;
constexpr uint32_t kImportEntries = 512;     // allocations one rank can export to processes that are its peers
constexpr uint32_t kWordEntryNull = 0xFFFF;  // exchange == 2: no buffer
constexpr uint32_t kWordEntryHeap = 0xFFFE;  // exchange == 2: the offset is one into the rank's heap
constexpr uint64_t kCreditOff = 12288;       // [kMaxCtas][kMaxRanks] u32: chunks a reducer has consumed (staged reduce)
constexpr int kStatusOutOfBounds = 14;       // MegRay::MEGRAY_OUT_OF_BOUNDS
// Small-message (flagged word) slots follow the pad: [2 parities][kMaxRanks sources] slots, each
// holding kLLMaxBytes of payload as 8-byte {data, flag} words.
constexpr uint64_t kLLMaxBytes = 1024 * 1024;
constexpr uint64_t kLLSlotBytes = 2 * kLLMaxBytes;
constexpr uint64_t kLLRegionBytes = 2 * kMaxRanks * kLLSlotBytes;  // 32 MiB

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
    uint64_t heap_bytes;   // size of every rank's heap
    int phases;            // 1: CTA 0 stamps %globaltimer at every phase boundary (pad, kPhaseOff)
    uint32_t spin_sleep_ns;  // pause between the polls of a wait that has lasted a while (0: none)
    // Extents of this call's buffers, for builds with MEGRAY_DEBUG_BOUNDS: every CTA-level copy or
    // reduction first checks that the range it is about to touch lies in some rank's heap or in
    // one of these buffers; a range that does not is skipped and recorded (pad, kDebugOff) and
    // the status word becomes MEGRAY_OUT_OF_BOUNDS.  0 = extent unknown (nothing may touch it).
    const void* guard_in;
    const void* guard_out;
    uint64_t guard_in_bytes;
    uint64_t guard_out_bytes;
    uint64_t guard_peer_in_bytes;   // exchanged buffers: what a peer's input / output holds
    uint64_t guard_peer_out_bytes;
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
//   broadcast       barrier; the message is cut into n-1 slices, one per non-root rank: the root
//                   stores slice j into rank j's output chunk by chunk and bumps a chunk counter
//                   there; rank j forwards each chunk of its slice, as it lands, to the outputs of
//                   the other non-root ranks.  The root sends the message once, every other rank
//                   receives it once and forwards 1/(n-1) of it: all links are busy at once.
//   reduce          barrier; rank r loads slice r of all inputs, combines, stores into the root's
//                   output; barrier.
//   gather          barrier; store this rank's block into slot r of the root's output; barrier.
//   scatter         barrier; the root stores chunk q of its input into rank q's output; barrier.
//
// Whose buffers?  Ranks that are threads of one process (the way the reference's tests and its
// benchmark drive their ranks) can address each other's cudaMalloc memory once peer access is
// on, so with `exchange` set every rank publishes the addresses of this call's buffers in the
// peers' pads as part of the first barrier and reads the peers' addresses from its own pad: plain
// unregistered user buffers then take these kernels.  Without `exchange` the host fills
// in_base / out_base (symmetric-heap or registered buffers).
enum DirectKind : int {
    DIRECT_ALL_REDUCE = 0,
    DIRECT_REDUCE_SCATTER = 1,
    DIRECT_ALL_GATHER = 2,
    DIRECT_ALL_TO_ALL = 3,
    DIRECT_BROADCAST = 4,
    DIRECT_REDUCE = 5,
    DIRECT_GATHER = 6,
    DIRECT_SCATTER = 7
};

struct DirectArgs {
    CommonArgs c;
    int kind;
    // every rank's input (all_reduce, reduce_scatter) and output (all_reduce, all_gather,
    // all_to_all) buffer as mapped in this rank's address space: heap addresses, or peer mappings
    // of buffers registered with the communicator
    const char* in_base[kMaxRanks];
    char* out_base[kMaxRanks];
    const void* in_local;  // this rank's input when only this rank reads it (any device memory), or,
                           // with `exchange`, the input this rank publishes
    void* out_local;       // likewise for the output
    uint64_t len;          // all_reduce / broadcast / reduce: total elements; others: elements per rank
    float scale;
    MegRay::DType in_dtype;
    MegRay::DType out_dtype;
    MegRay::ReduceOp op;
    char* mc_base;         // non-null: multicast (NVLS) mapping of the heap, use multimem
    int exchange;          // 1: in_word / out_word (this rank's buffer addresses) are published to the peers
                           // and theirs are read; 2: the words are (allocation entry << 48 | offset)
                           // and import_table maps (rank, entry) to the allocation's address here
    uint64_t in_word, out_word;
    const uint64_t* import_table;  // [kMaxRanks ranks][kImportEntries]; 0: not mapped yet, 1: cannot be mapped
    int parity;            // exchange: which of the two address slots this launch uses (alternates)
    int root;              // broadcast, reduce, gather, scatter
    uint64_t heap_bytes;   // size of every rank's heap (NVLS needs both buffers inside it, same offset)
    uint32_t chunk_base;   // broadcast: chunk k is announced as chunk_base + k + 1
    uint32_t chunk_bytes;  // broadcast: bytes of one chunk of a CTA's share of a slice (multiple of 16)
    int bcast_pull;        // broadcast by loads alone: every rank loads its slice from the root and the
                           // other slices from their owners (instead of the root and the owners storing)
    // reduce with the root's input pushed (stage_slots > 0): CTA b of the root stores chunk k of
    // every slice into slot (b * stage_slots + k % stage_slots) of chunk_bytes at stage_off in the
    // heap of the rank that reduces the slice
    uint64_t stage_off;
    uint32_t stage_slots;
    // 1: as above.  2: loads only - the reducer of a slice loads it from every rank and stores the
    // reduced chunks into slots in its OWN heap, and the root loads them from there into its output.
    int reduce_mode;
};

// Small messages: flagged words ("LL").  A sender stores every 4 bytes of payload together with
// the call's sequence number as one 8-byte word into the receiver's slot; the receiver polls the
// words themselves until they carry the sequence number.  No barrier and no memory fence stands
// between the data and its arrival, so a call costs one kernel launch plus one NVLink store
// latency.  Slots alternate between two parities; a slot is reused two calls later, when its
// reader has finished (every rank hears from every other rank in every call: through the payload
// itself, or, for rooted operations, through a token word).
struct LLArgs {
    CommonArgs c;
    uint32_t seq;                    // this call's flag value (never 0)
    uint64_t slot_off;               // heap offset of this parity's slots; slot of source q at + q * kLLSlotBytes
    uint64_t token_off;              // heap offset of this parity's token words [kMaxRanks] x 8 bytes
    const void* in;
    void* out;
    uint64_t bytes;                  // payload bytes per (source, destination) pair, <= kLLMaxBytes
    uint32_t send_mask;              // bit j: this rank sends `bytes` from in + send_off[j] to rank j
    uint32_t recv_mask;              // bit q: this rank consumes the payload rank q sent
    int64_t send_off[kMaxRanks];
    int64_t recv_off[kMaxRanks];     // copy mode: where source q's payload goes in `out`
    int self;                        // this rank's own part takes part: copy in + send_off[rank] -> out +
                                     // recv_off[rank], or (reduce) the operand at in + send_off[rank]
    int reduce;                      // 1: out[0, bytes) = op over the sources (and self) in rank order
    int tokens;                      // 1: exchange tokens (rooted operations)
    float scale;
    MegRay::DType in_dtype;
    MegRay::DType out_dtype;
    MegRay::ReduceOp op;
};
cudaError_t launch_ll(const LLArgs& args, int ctas, int threads, cudaStream_t stream);


// How the pipelined broadcast cuts a message of `bytes` bytes for n ranks and `ctas` CTAs: n - 1
// slices (one per non-root rank), every CTA owns `per_cta` bytes of each slice and moves them in
// `chunks` chunks of `chunk_bytes`.  Host and device compute it alike; the host advances the
// chunk sequence by `chunks` per call.
struct BcastPlan {
    uint64_t slice;    // bytes of one slice (multiple of 16)
    uint64_t per_cta;  // bytes of a slice one CTA moves (multiple of 16)
    uint32_t chunks;
};
__host__ __device__ inline BcastPlan bcast_plan(uint64_t bytes, int n, int ctas, uint32_t chunk_bytes) {
    BcastPlan p;
    const uint64_t ns = n > 1 ? static_cast<uint64_t>(n - 1) : 1;
    p.slice = ((bytes + ns - 1) / ns + 15) / 16 * 16;
    p.per_cta = ((p.slice + ctas - 1) / ctas + 15) / 16 * 16;
    p.chunks = static_cast<uint32_t>((p.per_cta + chunk_bytes - 1) / chunk_bytes);
    if (p.chunks == 0)
        p.chunks = 1;
    return p;
}

// The staged reduce: n - 1 slices of `slice` elements (one per non-root rank), of which every
// CTA takes `per_cta` elements in `chunks` chunks of `chunk_el` elements.
struct ReducePlan {
    uint64_t slice;
    uint64_t per_cta;
    uint64_t chunk_el;
    uint32_t chunks;
};
__host__ __device__ inline ReducePlan reduce_plan(uint64_t len, int n, int ctas, uint32_t chunk_bytes, uint32_t elem_bytes) {
    ReducePlan p;
    const uint64_t ns = n > 1 ? static_cast<uint64_t>(n - 1) : 1;
    const uint64_t v = 16 / elem_bytes;  // elements per 16-byte vector
    p.slice = ((len + ns - 1) / ns + v - 1) / v * v;
    p.per_cta = ((p.slice + ctas - 1) / ctas + v - 1) / v * v;
    p.chunk_el = chunk_bytes / elem_bytes;
    p.chunks = static_cast<uint32_t>((p.per_cta + p.chunk_el - 1) / p.chunk_el);
    if (p.chunks == 0)
        p.chunks = 1;
    return p;
}

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
