// Endpoint over reliable-connected RDMA queue pairs: one-sided read / write / write-with-immediate,
// immediate receive, and two-sided send / recv by rendezvous.
//
// Three channels per endpoint: `io` (num_qp queue pairs, one-sided traffic), `msg` (num_qp queue
// pairs, payload of send / recv) and `meta` (one queue pair, 64-byte inline control messages).
//
// One-sided path. An operation becomes per-lane lists of work requests: every assignment is cut into
// chunks of at most SLIME_MAX_LENGTH_PER_ASSIGNMENT; a chunk of at least SLIME_STRIPE_MIN_BYTES is
// striped over all lanes, a smaller one goes whole to one lane (round robin) so that small transfers
// do not pay num_qp doorbells. Every 32nd work request of a lane and its last one are signaled. The
// progress thread posts from a FIFO: the head waits for its buffers to be ready on the stream and
// for per-lane send credits (SLIME_MAX_SEND_WR, refunded by signaled completions); a batch larger
// than the credit is posted in pieces. Completion callbacks OR the lane into the operation's mask.
//
// write_with_imm. Ordering holds only inside a queue pair, so the immediate is sent on EVERY lane,
// after that lane's data (on the lane's last data work request, or a zero-length one): the receiver
// hands the k-th event to the application when the k-th immediate has arrived on all lanes, which is
// when all stripes have landed. A window of SLIME_MAX_IO_FIFO_DEPTH zero-length receives stays posted
// per lane and is refilled from the completion thread.
//
// send / recv. recv(k) announces {address, key, length} in a meta message once the buffer is ready;
// send(k) waits for the k-th announcement, then writes the payload striped over the msg lanes with
// the same all-lanes immediate; the receiver completes recv(k) on the k-th immediate group. Sends and
// receives must be issued in the same relative order on the two sides.
//
// Memory regions are registered in the pool of the device context, shared by all endpoints on that device.
//
// Same API, status codes and environment knobs as the reference's RDMAEndpoint
// (dlslime/csrc/engine/rdma/rdma_endpoint.h:203-259, rdma_endpoint.cpp:689-850,1044-1337 in the
// reference); the all-lanes immediate and the small-transfer rule are this implementation's own.
#pragma once

#include <atomic>
#include <deque>
#include <mutex>
#include <optional>
#include <unordered_map>
#include <vector>

#include "core/ring.h"
#include "transport/endpoint.h"
#include "transport/rdma/rdma_context.h"

namespace slime {
namespace rdma {

class RdmaWorker;

class RdmaEndpoint final: public Endpoint, public CompletionSink, public std::enable_shared_from_this<RdmaEndpoint> {
public:
    // device "" = first device; link_type "RoCE" | "IB" | "". num_qp <= 0 takes SLIME_QP_NUM.
    static std::shared_ptr<RdmaEndpoint> create(const std::string& device = "", int port = 1, const std::string& link_type = "",
                                                int num_qp = 0);
    // On an existing context, progressed by `worker` (nullptr = the shared worker of the context's NUMA node).
    static std::shared_ptr<RdmaEndpoint> create(std::shared_ptr<RdmaContext> ctx, int num_qp, std::shared_ptr<RdmaWorker> worker);
    // Hands the endpoint to another progress worker (nullptr = back to the shared worker of its NUMA node).
    void set_worker(std::shared_ptr<RdmaWorker> worker);
    ~RdmaEndpoint() override;

    std::string kind() const override { return "rdma"; }
    Json        endpoint_info() override;
    int         connect(const Json& remote_info) override;
    bool        connected() const override { return connected_.load(); }

    std::shared_ptr<ReadWriteFuture> read(const std::vector<assign_tuple_t>& assign, void* stream = nullptr) override;
    std::shared_ptr<ReadWriteFuture> write(const std::vector<assign_tuple_t>& assign, void* stream = nullptr) override;
    std::shared_ptr<ReadWriteFuture> write_with_imm(const std::vector<assign_tuple_t>& assign, int32_t imm_data,
                                                    void* stream = nullptr) override;
    std::shared_ptr<ImmRecvFuture>   imm_recv(void* stream = nullptr) override;
    std::shared_ptr<SendFuture>      send(const chunk_tuple_t& chunk, void* stream = nullptr) override;
    std::shared_ptr<RecvFuture>      recv(const chunk_tuple_t& chunk, void* stream = nullptr) override;

    void shutdown() override;
    void cancel_all() override;
    int  process() override;

    void on_completion(const Completion& wc) override;

    int                                 num_qp() const { return num_qp_; }
    const std::shared_ptr<RdmaContext>& context() const { return ctx_; }
    // Counters for tests and tuning.
    uint64_t posted_wrs() const { return posted_wrs_.load(); }
    uint64_t signaled_wrs() const { return signaled_wrs_.load(); }
    uint64_t credit_stalls() const { return credit_stalls_.load(); }

private:
    RdmaEndpoint(std::shared_ptr<RdmaContext> ctx, int num_qp);

    enum ChannelId : int { CH_IO = 0, CH_MSG = 1, CH_META = 2 };
    enum WrKind : uint64_t { K_TX = 1, K_TX_UNSIGNALED = 2, K_WINDOW_RECV = 3, K_META_SEND = 4, K_META_RECV = 5 };
    static uint64_t make_wr_id(WrKind kind, uint32_t refund, uint32_t index)
    {
        return (static_cast<uint64_t>(kind) << 60) | (static_cast<uint64_t>(refund & 0xffff) << 40) | index;
    }

    struct Lane {
        uint64_t         qp  = 0;
        uint32_t         qpn = 0;
        uint32_t         psn = 0;
        std::atomic<int> credits{0};
        std::deque<uint32_t> imms;  // immediates that arrived on this lane, oldest first (imm_mu_)
        Lane() = default;
        Lane(Lane&& o) noexcept: qp(o.qp), qpn(o.qpn), psn(o.psn), credits(o.credits.load()), imms(std::move(o.imms)) {}
    };
    struct Channel {
        std::vector<Lane> lanes;
        int               recv_window = 0;
    };

    // One lane's share of one operation while it is in flight.
    struct TxLane {
        std::shared_ptr<EndpointOpState> state;
        int                              lane    = 0;
        int                              channel = 0;
        std::atomic<int>                 outstanding{0};  // signaled work requests not yet completed
    };
    struct TxOp {
        std::shared_ptr<EndpointOpState>  state;
        int                               channel = CH_IO;
        std::vector<std::vector<SendWr>>  lane_wrs;
        std::vector<size_t>               cursor;
        std::vector<int32_t>              slot;  // TxLane slot per lane, -1 until leased
        bool                              leased = false;
    };
    struct MetaMsg {  // 64 bytes on the wire
        uint64_t seq;
        uint64_t addr;
        uint64_t length;
        uint32_t rkey;
        uint32_t pad[9];
    };
    struct RecvOp {
        std::shared_ptr<EndpointOpState> state;
        uintptr_t                        addr   = 0;
        uint64_t                         length = 0;
        uint32_t                         rkey   = 0;
        uint64_t                         seq    = 0;
    };
    struct SendOp {
        std::shared_ptr<EndpointOpState> state;
        uintptr_t                        addr   = 0;
        uint64_t                         length = 0;
        uint32_t                         lkey   = 0;
    };

    void     init_channel(Channel& ch, int lanes, const QpCaps& caps);
    int      connect_channel(Channel& ch, const Json& remote, const char* name);
    void     post_window(Channel& ch, int channel_id);
    void     build_striped(TxOp& op, WrOp data_op, uint64_t local_addr, uint32_t lkey, uint64_t remote_addr, uint32_t rkey,
                           uint64_t length, size_t& rr);
    void     finish_lanes(TxOp& op, bool with_imm, uint32_t imm);
    std::shared_ptr<ReadWriteFuture> submit_one_sided(OpCode opcode, const std::vector<assign_tuple_t>& assign, int32_t imm, void* stream);
    int      post_tx(int channel_id);
    int      progress_recv();
    int      progress_send();
    void     lane_done(TxLane& tl, uint32_t slot);
    void     fail_tx(TxOp& op);
    void     complete_state(const std::shared_ptr<EndpointOpState>& st);
    void     deliver_group(int channel_id, uint32_t imm);
    void     repost_window(int channel_id, int lane);
    bool     ensure_local(uintptr_t addr, uint64_t bytes, MemoryRegion& out);
    void     wake_worker();

    std::shared_ptr<RdmaContext> ctx_;
    std::shared_ptr<RdmaWorker>  worker_;
    std::shared_ptr<LocalMemoryPool> own_pool_;  // the context's shared pool (local_pool_ may be replaced by set_local_pool)
    std::string                      meta_name_;
    int                          num_qp_ = 1;
    Channel                      ch_[3];
    std::atomic<bool>            connected_{false}, shut_{false};
    uint64_t                     stripe_min_bytes_ = 64 << 10;

    // submit FIFOs (user threads -> progress thread)
    std::mutex          fifo_mu_;
    std::deque<TxOp>    tx_fifo_[2];
    std::optional<TxOp> cur_tx_[2];       // head operation being posted (proc_mu_)
    std::mutex          proc_mu_;         // process() against cancel_all() / shutdown()
    std::deque<RecvOp>  recv_fifo_;       // not yet announced
    std::deque<SendOp>  send_fifo_;
    size_t              rr_lane_ = 0;     // round robin for unstriped chunks (fifo_mu_)
    uint64_t            recv_seq_ = 0;

    // operations submitted and not yet settled, for cancel_all (weak: the futures own the state)
    std::mutex                                                            inflight_mu_;
    std::unordered_map<EndpointOpState*, std::weak_ptr<EndpointOpState>> inflight_;
    void track(const std::shared_ptr<EndpointOpState>& st);

    // in-flight lane slots
    std::vector<TxLane>  tx_slots_;
    MpmcRing<uint32_t>   free_slots_;

    // immediate events and rendezvous state (completion thread <-> users / progress thread)
    std::mutex                                   imm_mu_;
    std::deque<std::shared_ptr<EndpointOpState>> imm_waiters_;
    std::deque<uint32_t>                         imm_events_;
    std::deque<RecvOp>                           announced_;  // recvs whose meta went out, oldest first
    std::deque<MetaMsg>                          metas_;      // announcements received, oldest first

    // meta ring: receive slots then send staging, one registered buffer
    std::vector<uint8_t> meta_buf_;
    MemoryRegion         meta_mr_;
    int                  meta_depth_ = 0;

    std::atomic<uint64_t> posted_wrs_{0}, signaled_wrs_{0}, credit_stalls_{0};
};

}  // namespace rdma
}  // namespace slime
