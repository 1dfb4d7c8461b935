// Native NVLink 5 / NVSwitch backend (Backend MEGRAY_NVL).
//
// Every collective is one kernel launch per rank on the caller's stream: the
// kernels in kernels/collectives.cu move data through a symmetric heap that all
// ranks map, synchronise through flag words in that heap, and fuse the
// reduction, scale and cast into the transfer.  User buffers need no
// registration: inputs are pushed into peers' staging slots (or published in
// the local heap) and results are loaded from peers' heaps straight into the
// output.  send/recv and group_start/group_end go to NCCL point-to-point.
//
// Replaces, behind the same interface, what the reference does through
// ncclAllReduce & co. (src/nccl/communicator.cpp:90-228).
#pragma once
#include <cuda_runtime_api.h>

#include <map>
#include <memory>
#include <vector>

#include "kernels/collectives.cuh"
#include "megray/communicator.h"
#include "megray/fused.h"
#include "megray/server.h"
#include "nvl/sym_heap.h"

namespace MegRay {

class IpcCache;

class NcclCommunicator;

class NvlCommunicator : public Communicator, public NvlInterface {
public:
    NvlCommunicator(uint32_t nranks, uint32_t rank);
    ~NvlCommunicator() override;

    Status do_init() override;
    Status do_init(BcastCallback cb) override;

    Status scatter(const void* sendbuff, void* recvbuff, size_t recvlen, DType dtype, uint32_t root,
                   std::shared_ptr<Context> ctx) override;
    Status gather(const void* sendbuff, void* recvbuff, size_t sendlen, DType dtype, uint32_t root,
                  std::shared_ptr<Context> ctx) override;
    Status all_to_all(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                      std::shared_ptr<Context> ctx) override;
    Status all_gather(const void* sendbuff, void* recvbuff, size_t sendlen, DType dtype,
                      std::shared_ptr<Context> ctx) override;
    Status all_reduce(const void* sendbuff, void* recvbuff, size_t len, DType dtype, ReduceOp op,
                      std::shared_ptr<Context> ctx) override;
    Status reduce_scatter(const void* sendbuff, void* recvbuff, size_t recvlen, DType dtype,
                          ReduceOp op, std::shared_ptr<Context> ctx) override;
    Status broadcast(const void* sendbuff, void* recvbuff, size_t len, DType dtype, uint32_t root,
                     std::shared_ptr<Context> ctx) override;
    Status reduce(const void* sendbuff, void* recvbuff, size_t len, DType dtype, ReduceOp op,
                  uint32_t root, std::shared_ptr<Context> ctx) override;
    Status group_start() override;
    Status group_end() override;

    Backend backend() const override { return MEGRAY_NVL; }
    void abort() override;
    Status status() override;
    CommStats stats() override;

    // NvlInterface
    void* sym_alloc(size_t bytes, size_t* offset_out) override;
    Status sym_free(void* ptr) override;
    void* peer_ptr(void* ptr, uint32_t peer) override;
    bool in_heap(const void* ptr, size_t bytes) override;
    size_t heap_bytes() override { return m_heap.bytes(); }
    void* heap_base(uint32_t peer) override { return m_heap.base(peer); }
    Status register_buffer(void* ptr, size_t bytes) override;
    Status deregister_buffer(void* ptr) override;
    Status all_reduce_scaled(const void* sendbuff, void* recvbuff, size_t len, DType in_dtype,
                             DType out_dtype, float scale, ReduceOp op,
                             std::shared_ptr<Context> ctx) override;
    Status stream_barrier(std::shared_ptr<Context> ctx) override;
    Status check_canaries() override;
    int read_phase_stamps(uint64_t* out, int max) override;
    void set_p2p_async(bool on) override { m_p2p_async = on; }
    Status p2p_join(std::shared_ptr<Context> ctx) override;
    Status fused_begin(void* stream) override;
    void fused_end(void* stream) override;
    uint32_t fused_call_count(const void* flags) override;
    void ll_ticket(uint32_t* seq, size_t* slot_off, size_t* slot_stride) override;
    uint32_t reserve_epochs(uint32_t count) override;
    size_t fused_flag_offset() override { return kFusedFlagOff; }
    int* status_word() override { return m_status_dev; }
    uint64_t device_timeout_ns() override { return m_timeout_ns; }
    void set_device_timeout_ms(int64_t ms) override { m_timeout_ns = static_cast<uint64_t>(ms) * 1000000ull; }

    // heap layout (byte offsets, identical on every rank)
    static constexpr size_t kFlagOff = mgk::coll::kBarrierFlagOff;  // collectives: first 16 KiB of the pad
    static constexpr size_t kFusedFlagOff = 16 * 1024;              // fused kernels: 48 KiB of flags/counters
    static constexpr size_t kLLOff = mgk::coll::kPadBytes;          // small-message slots (32 MiB)
    static constexpr size_t kWorkspaceOff = mgk::coll::kPadBytes + mgk::coll::kLLRegionBytes;  // two staging workspaces

protected:
    Status _send(const void* sendbuff, size_t size, uint32_t rank,
                 std::shared_ptr<Context> ctx) override;
    Status _recv(void* recvbuf, size_t size, uint32_t rank, std::shared_ptr<Context> ctx) override;

private:
    enum class ReduceKind { AllReduce, Reduce, ReduceScatter };
    Status begin(const std::shared_ptr<Context>& ctx, cudaStream_t* stream);
    Status begin_on(cudaStream_t stream);  // state checks + cross-stream ordering
    Status reduce_impl(ReduceKind kind, const void* in, void* out, size_t len, DType in_dtype,
                       DType out_dtype, float scale, ReduceOp op, uint32_t root,
                       cudaStream_t stream);
    mgk::coll::CommonArgs common_args(uint32_t epochs = 2);
    size_t workspace_off();  // offset of the workspace this launch uses; flips the parity
    // Guard zones of kCanaryBytes, filled with kCanaryByte at init, lie before, between and after
    // the two staging workspaces; nothing ever writes there, and check_canaries() verifies it.
    static constexpr size_t kCanaryBytes = 4096;
    static constexpr unsigned char kCanaryByte = 0xC5;
    size_t canary_off(int zone) const;
    void after_launch(cudaStream_t stream);
    void adopt_device_status();
    int pick_ctas(size_t bytes) const;
    bool aligned_heap(const void* p, size_t bytes);
    // A user buffer registered with register_buffer(): this rank's range and every rank's twin.
    struct Registration {
        char* local = nullptr;
        size_t bytes = 0;
        char* peer[mgk::coll::kMaxRanks] = {};
        std::vector<void*> ipc_bases;  // mappings opened for this registration (other processes)
    };
    // Fills base[q] with rank q's twin of [p, p + bytes) when p is 16-byte aligned and lies in
    // the symmetric heap or in a registered range; `heap_off` receives the heap offset or
    // SIZE_MAX for a registered buffer.
    bool peer_view(const void* p, size_t bytes, char** base, size_t* heap_off);
    void drop_registration(Registration& r);
    Status direct_launch(int kind, const void* in, void* out, size_t len, DType in_dtype, DType out_dtype,
                         float scale, ReduceOp op, cudaStream_t stream);
    // Single-pass kernel on this call's buffers as they are (ranks of one process: addresses travel
    // through the pads).  `in_bytes` / `out_bytes`: what this rank reads / writes of its own
    // buffers; `in_shared` / `out_shared`: the peers' kernels touch that buffer too, so it must be
    // memory they can address (otherwise it is replaced by a bounce buffer for this call).
    Status exchange_launch(int kind, const void* in, size_t in_bytes, bool in_shared, void* out, size_t out_bytes,
                           bool out_shared, size_t len, DType in_dtype, DType out_dtype, float scale, ReduceOp op,
                           uint32_t root, cudaStream_t stream);
    // Small-message kernel; `a` comes filled with the operation's send / receive pattern.
    Status ll_launch(mgk::coll::LLArgs& a, cudaStream_t stream);
    Status p2p_call(bool is_send, void* buf, size_t size, uint32_t rank, const std::shared_ptr<Context>& ctx);
    Status p2p_fork(cudaStream_t user);
    Status p2p_finish();
    bool peer_addressable(const void* p, size_t bytes);
    bool exchange_fits(const void* in, size_t in_bytes, const void* out, size_t out_bytes);
    // extents of the current call's buffers, handed to the kernels (see CommonArgs::guard_in)
    void set_guard(const void* in, size_t in_bytes, void* out, size_t out_bytes);
    void* bounce(int which, size_t bytes);
    size_t ll_limit(int kind) const { return m_ll_bytes[kind]; }
    Status check_cuda(cudaError_t e);

    SymmetricHeap m_heap;
    std::unique_ptr<Server> m_own_server;  // init(BcastCallback): private rendezvous
    std::unique_ptr<NcclCommunicator> m_p2p;
    // send / recv: a stream of the communicator's own, forked from and joined to the caller's
    cudaStream_t m_p2p_stream = nullptr;
    cudaEvent_t m_p2p_fork = nullptr, m_p2p_done = nullptr;
    std::shared_ptr<Context> m_p2p_ctx;
    std::vector<cudaStream_t> m_p2p_users;  // callers' streams of the open group
    bool m_p2p_grouping = false;
    bool m_p2p_async = false;
    bool m_p2p_pending = false;
    bool m_ready = false;
    size_t m_ws_bytes = 0;   // bytes of one staging workspace
    size_t m_user_off = 0;   // first byte of the symmetric allocator's area
    size_t m_user_top = 0;   // bump pointer
    std::vector<size_t> m_allocs;
    std::vector<Registration> m_regs;
    std::map<size_t, uint32_t> m_fused_calls;  // heap offset of a fused counter block -> calls so far
    uint32_t m_epoch = 0;
    int m_parity = 0;
    uint64_t m_timeout_ns;
    int m_max_ctas;
    size_t m_oneshot_bytes;
    size_t m_nvls_min_bytes = 0;
    size_t m_cta_bytes = 128 * 1024;  // message bytes per CTA when sizing a collective's grid
    size_t m_direct_cta_bytes = 32 * 1024;  // the same for the single-pass kernels
    bool m_direct = true;
    // Ranks that are threads of one process, with peer access enabled between all their devices:
    // every collective above the small-message limit runs the single-pass kernels on the user's
    // buffers (MEGRAY_EXCHANGE=0 turns it off).
    struct {
        const void* in = nullptr;
        size_t in_bytes = 0;
        void* out = nullptr;
        size_t out_bytes = 0;
        // extents of the peers' buffers of the same call: the declared sizes, also on a rank
        // that passes no buffer of its own (the non-root ranks of a rooted operation)
        size_t peer_in_bytes = 0;
        size_t peer_out_bytes = 0;
    } m_guard;
    bool m_guard_shrink = false;
    bool m_phases = false;  // MEGRAY_PHASES=1: kernels stamp %globaltimer at their phase boundaries
    bool m_xchg = false;
    std::unique_ptr<IpcCache> m_ipc;  // ranks in separate processes: export logs and import table
    int m_xchg_parity = 0;
    uint32_t m_ll_seq = 0;      // small-message calls so far
    int m_ll_parity = 0;
    // all_reduce between the small-message limit and the one-shot limit: one-shot through the
    // staging slots (one barrier) rather than the single-pass kernel (two)
    bool m_oneshot_first = true;
    uint32_t m_chunk_seq = 0;   // chunks announced by pipelined broadcasts so far
    uint32_t m_bcast_chunk = 128 * 1024;
    // reduce of at least this many bytes: the root pushes its input (MEGRAY_REDUCE_STAGED_MIN / tune
    // table "reduce_staged_min_bytes")
    size_t m_reduce_staged_min = 8u << 20;
    // how a large reduce on more than two ranks runs: 0 the reducers load everything and store to
    // the root, 1 the root pushes its input into the reducers' slots, 2 loads only (the root loads
    // the reduced chunks from the reducers' slots), 3 loads only in steps separated by barriers
    // (MEGRAY_REDUCE_STEPS pieces).  MEGRAY_REDUCE_MODE / tune table "reduce_mode".
    int m_reduce_mode = 0;
    // broadcast by loads alone from this size on (MEGRAY_BCAST_PULL, MEGRAY_BCAST_PULL_MIN / tune table
    // "bcast_pull", "bcast_pull_min_bytes")
    bool m_bcast_pull = false;
    size_t m_bcast_pull_min = 0;
    uint32_t m_spin_sleep_ns = 0;  // MEGRAY_SPIN_SLEEP_NS / tune table "spin_sleep_ns"
    // largest payload per (source, destination) pair that goes as flagged words, per DirectKind
    size_t m_ll_bytes[8] = {};
    void* m_bounce[2] = {nullptr, nullptr};
    size_t m_bounce_cap[2] = {0, 0};
    // all_gather / all_to_all of at most this many bytes per rank (per peer for all_to_all) take
    // the push form (stores into the peers' buffers before the barrier instead of loads from
    // them after it).  Measured: on 2 GPUs 9.0 vs 9.7-10.1 us at 1 KiB and 10.1-10.4 vs
    // 11.8-13.0 us at 16 KiB; on 8 GPUs 17.9-18.1 us at 1 KiB (push) against 39-44 us at 16 KiB
    // (pull).  MEGRAY_PUSH_EXCHANGE=0 turns it off.
    static constexpr size_t kPushExchangeBytes = 64 * 1024;
    bool m_push_exchange = true;
    int* m_status_host = nullptr;  // pinned, mapped
    int* m_status_dev = nullptr;
    cudaStream_t m_last_stream = nullptr;
    cudaEvent_t m_last_event = nullptr;
    bool m_has_last = false;
    Status m_error = MEGRAY_OK;
};

}  // namespace MegRay
