// Endpoint over TCP sockets for CPU ranks and hosts without RDMA or NVLink.
//
// Each endpoint listens on its own port. connect() dials the peer's listener; that
// outgoing connection carries this side's requests (and their responses), while the
// connection accepted from the peer is served against the local memory regions. Three
// threads per endpoint: sender (drains the submit queue), receiver (responses ->
// futures) and server (peer requests -> local memory, immediate events, send/recv
// matching). One-sided operations complete when the peer acknowledged the last piece.
//
// The reference has no TCP engine (it lists one as future work, docs/roadmap.md:27-30 in
// the reference); this one provides the full endpoint API so that every layer above
// (PeerAgent, RPC, cache) runs on any machine.
#pragma once

#include <atomic>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <thread>
#include <unordered_map>

#include "core/ring.h"
#include "transport/endpoint.h"

namespace slime {

class TcpEndpoint final: public Endpoint, public std::enable_shared_from_this<TcpEndpoint> {
public:
    explicit TcpEndpoint(const std::string& bind_host = "127.0.0.1", int port = 0, int num_lanes = 1);
    ~TcpEndpoint() override;

    std::string kind() const override { return "tcp"; }
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

    // The owner's handle is the key a request carries, whatever index the entry gets locally.
    int32_t register_remote_memory_region(const std::string& name, const Json& info) override
    {
        Json copy    = info;
        copy["rkey"] = static_cast<unsigned long long>(info["handle"].as_uint());
        return remote_pool_->register_remote_memory_region(name, copy);
    }

    void shutdown() override;
    void cancel_all() override;

    int         port() const { return port_; }
    std::string host() const { return host_; }

    // Test hooks (host-side fault injection): "drop_ack" swallows the next n acknowledgements,
    // "reset" closes the outgoing socket before the next n requests, "fail_write" makes the
    // server reject the next n writes.
    void inject_fault(const std::string& what, int count);

private:
    struct Op {
        OpCode                           opcode;
        std::vector<assign_tuple_t>      assign;
        chunk_tuple_t                    chunk{};
        int32_t                          imm = 0;
        std::shared_ptr<EndpointOpState> state;
        uint64_t                         id = 0;
    };
    struct PendingRecv {
        uintptr_t                        ptr;
        size_t                           length;
        std::shared_ptr<EndpointOpState> state;
    };

    std::shared_ptr<ReadWriteFuture> submit_one_sided(OpCode op, const std::vector<assign_tuple_t>& assign, int32_t imm, void* stream);
    void sender_loop();
    void receiver_loop();
    void acceptor_loop();
    void server_loop(int fd);
    bool post_op(Op& op);
    // Posts `op` on the calling thread when nothing is queued or being posted (small operations: no hand-over to the
    // sender thread, one wake-up less per operation). False = not taken, queue it.
    bool try_post_inline(Op& op, uint64_t bytes);
    void enqueue(Op&& op);
    void complete(const std::shared_ptr<EndpointOpState>& st, int32_t status);
    void fail_everything(int32_t status);
    void deliver_imm(int32_t imm);
    void deliver_message(std::vector<uint8_t>&& payload);

    std::string host_;
    int         port_      = 0;
    int         listen_fd_ = -1;
    int         out_fd_    = -1;
    int         obs_link_  = -1;
    std::atomic<bool> connected_{false}, stopping_{false}, shut_{false};
    std::atomic<uint64_t> next_id_{1};

    std::mutex              submit_mu_;
    std::condition_variable submit_cv_;
    std::deque<Op>          submit_q_;
    bool                    posting_ = false;  // under submit_mu_: some thread is inside post_op (operations leave in order)
    std::atomic<bool>       broken_{false};    // a post failed: the link is gone, later operations fail at once

    std::mutex                       inflight_mu_;
    std::unordered_map<uint64_t, Op> inflight_;  // awaiting an acknowledgement or read data

    std::mutex                                    imm_mu_;
    std::deque<std::shared_ptr<EndpointOpState>>  imm_waiters_;
    std::deque<int32_t>                           imm_events_;

    std::mutex                        msg_mu_;
    std::deque<PendingRecv>           recv_posted_;
    std::deque<std::vector<uint8_t>>  msg_unexpected_;

    std::mutex       out_write_mu_;
    std::thread      sender_, receiver_, acceptor_;
    std::mutex       servers_mu_;
    std::vector<std::thread> servers_;
    std::vector<int>         server_fds_;

    std::atomic<int> fault_drop_ack_{0}, fault_reset_{0}, fault_fail_write_{0};
};

}  // namespace slime
