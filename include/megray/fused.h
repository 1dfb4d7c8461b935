/**
 * Entry points of the native NVLink backend that go beyond the MegRay
 * interface: symmetric memory, the fused scale/cast all_reduce, and (declared
 * in the headers named below) the GEMM-fused and MoE collectives.  None of
 * these has a counterpart in the reference, whose interface ends at
 * include/megray/communicator.h:60-109.
 *
 * Obtain the interface from a communicator made with MEGRAY_NVL:
 *     auto comm = MegRay::get_communicator(n, r, MegRay::MEGRAY_NVL);
 *     auto* nvl = MegRay::as_nvl(comm.get());
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <memory>

#include "megray/communicator.h"

namespace MegRay {

class NvlInterface {
public:
    virtual ~NvlInterface() = default;

    /** Symmetric allocation: every rank must call with the same size in the same order.
     *  The returned pointer is device memory of this rank; peers reach it with peer_ptr().
     *  `offset_out` (optional) receives the offset inside the heap, equal on all ranks. */
    virtual void* sym_alloc(size_t bytes, size_t* offset_out = nullptr) = 0;
    /** Release the most recent allocations down to (and including) `ptr`: the allocator is a
     *  stack, which keeps offsets identical on all ranks without any communication. */
    virtual Status sym_free(void* ptr) = 0;
    /** Address, in this rank's address space, of `ptr`'s twin on rank `peer`. */
    virtual void* peer_ptr(void* ptr, uint32_t peer) = 0;
    /** True if [ptr, ptr+bytes) lies inside this rank's symmetric heap. */
    virtual bool in_heap(const void* ptr, size_t bytes) = 0;
    virtual size_t heap_bytes() = 0;
    /** Base address of rank `peer`'s heap as mapped here. */
    virtual void* heap_base(uint32_t peer) = 0;

    /**
     * Collective.  Makes [ptr, ptr + bytes), ordinary device memory of this rank (cudaMalloc, a
     * framework's caching allocator), directly reachable by the kernels of every peer, so that
     * collectives on it take the single-pass paths instead of staging through the heap.
     * Every rank calls it with its own buffer, in the same order; a collective then qualifies
     * when each rank passes an address at the same distance from the start of its registered
     * range.  Peers in the same process use the address as it is (peer access is enabled);
     * peers in other processes map it through a CUDA IPC handle, which exists for cudaMalloc
     * memory only: if any rank's memory has none, every rank gets MEGRAY_NOT_IMPLEMENTED and
     * the buffer keeps working through the staged paths.
     */
    virtual Status register_buffer(void* ptr, size_t bytes) = 0;
    /** Collective.  Drops the registration that starts at `ptr` (and this rank's mappings of
     *  the peers' buffers registered in the same call). */
    virtual Status deregister_buffer(void* ptr) = 0;

    /**
     * out = cast<out_dtype>(scale * reduce_op(in over ranks)): the gradient-bucket path.
     * Floating dtypes (fp16, bf16, fp32; fp64 with out_dtype == in_dtype); scale applies to SUM.
     */
    virtual Status all_reduce_scaled(const void* sendbuff, void* recvbuff, size_t len,
                                     DType in_dtype, DType out_dtype, float scale, ReduceOp op,
                                     std::shared_ptr<Context> ctx) = 0;

    /**
     * send / recv run on a stream of the communicator's own, ordered after the work already on the
     * caller's stream.  By default the caller's stream then waits for the transfer (the calls
     * complete in stream order, as the interface says).  With set_p2p_async(true) that wait is
     * postponed to p2p_join(ctx): whatever the caller enqueues in between, native collectives
     * included, overlaps the transfer, and must not touch the buffers in flight.
     */
    virtual void set_p2p_async(bool on) = 0;
    /** Makes ctx's stream wait for every send / recv issued so far (no-op when none is pending). */
    virtual Status p2p_join(std::shared_ptr<Context> ctx) = 0;

    /** With MEGRAY_PHASES=1 in the environment the collective kernels stamp %globaltimer (ns) at
     *  their phase boundaries (block 0 of this rank).  Synchronises the device and copies the
     *  stamps of the most recent kernel into `out` (at most `max`); returns how many there are.
     *  Single-pass kernels: start, first barrier passed, data moved, last barrier passed.
     *  Flagged-word kernel: start, all sent, all received.  Staged reduce kernel: start, pushed,
     *  barrier, reduced, barrier, gathered. */
    virtual int read_phase_stamps(uint64_t* out, int max) = 0;

    /** Synchronises the device and verifies the guard zones around the staging workspaces (filled
     *  with a pattern at init; no kernel may write there).  MEGRAY_OUT_OF_BOUNDS if one was touched. */
    virtual Status check_canaries() = 0;

    /** Barrier on the stream: later work of every rank starts after earlier work of all ranks. */
    virtual Status stream_barrier(std::shared_ptr<Context> ctx) = 0;

    /** What every collective of this communicator does before its launch, for fused entry points
     *  of other modules (the GEMM-fused tensor-parallel calls): refuses with the communicator's
     *  state when it is not initialised, aborted or failed (a kernel wait that ran out earlier),
     *  and orders `stream` after the communicator's previous launch on another stream. */
    virtual Status fused_begin(void* stream) = 0;
    /** Records that a kernel using the communicator's flags was launched on `stream`. */
    virtual void fused_end(void* stream) = 0;
    /** How many fused calls have used the counter block at `flags` (symmetric-heap memory),
     *  this one included.  The count belongs to the communicator and to the allocation: it
     *  starts again from 1 after sym_free of that memory or for a new communicator, which is
     *  when the counters themselves are zero again. */
    virtual uint32_t fused_call_count(const void* flags) = 0;

    /** Reserves the small-message slots of the next call for a kernel of another module (every
     *  rank must do so in the same order as its other calls): `seq` is the flag value its words
     *  carry, the slot of source rank q starts at heap + slot_off + q * slot_stride. */
    virtual void ll_ticket(uint32_t* seq, size_t* slot_off, size_t* slot_stride) = 0;

    /** Next flag epoch for kernels of other modules that synchronise through the pad
     *  (`count` consecutive values are reserved). */
    virtual uint32_t reserve_epochs(uint32_t count) = 0;
    /** Byte offset, inside every heap, of a flag area reserved for fused kernels. */
    virtual size_t fused_flag_offset() = 0;
    /** Device-visible status word of this communicator (0 = ok). */
    virtual int* status_word() = 0;
    /** Limit of one in-kernel wait, in nanoseconds. */
    virtual uint64_t device_timeout_ns() = 0;
    /** Override it (tests of the timeout path use a short limit). */
    virtual void set_device_timeout_ms(int64_t ms) = 0;
};

/** The NVL interface of `comm`, or nullptr if it is another backend. */
NvlInterface* as_nvl(Communicator* comm);

}  // namespace MegRay
