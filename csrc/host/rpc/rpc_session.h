// SlimeRPC session: request / reply over slotted mailboxes written with one-sided
// write-with-immediate. Wire format (kept from the reference, dlslime/csrc/rpc/rpc_constants.h:8-56
// in the reference): a slot holds [u32 tag | u32 total_len incl. header | u64 request_id | payload],
// the immediate value is the slot index, a request written to server slot s is answered in
// client slot s, and tag carries flag bits EXC 1<<27, ACK 1<<28, REPLY 1<<29, CHUNK 1<<30,
// LAST 1<<31. WIRE_VERSION = 3.
//
// The session works over any Endpoint (TCP or RDMA). Two modes: a receive pump thread that
// demultiplexes replies to futures and requests to an inbox, or pump-less single flight where
// call() itself waits for the reply (lowest latency for a client with one slot).
#pragma once

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>

#include "transport/endpoint.h"

namespace slime {
namespace rpc {

constexpr uint32_t WIRE_VERSION = 3;
#pragma pack(push, 1)
struct WireHeader {
    uint32_t tag;
    uint32_t total_len;
    uint64_t request_id;
};
#pragma pack(pop)
static_assert(sizeof(WireHeader) == 16, "the wire header is exactly 16 bytes");
constexpr size_t   HEADER_SIZE    = sizeof(WireHeader);
constexpr uint32_t EXC_BIT        = 1u << 27;
constexpr uint32_t ACK_BIT        = 1u << 28;
constexpr uint32_t REPLY_BIT      = 1u << 29;
constexpr uint32_t CHUNK_BIT      = 1u << 30;
constexpr uint32_t LAST_BIT       = 1u << 31;
constexpr uint32_t FLAG_MASK      = REPLY_BIT | EXC_BIT | ACK_BIT | CHUNK_BIT | LAST_BIT;
constexpr uint32_t MAX_SLOT_COUNT = 1u << 16;

class ClientFuture {
public:
    ClientFuture(uint64_t request_id, uint32_t slot_id): request_id_(request_id), slot_id_(slot_id) {}

    // Blocks until the reply arrived (or the session failed). Returns false on timeout (timeout_ms >= 0).
    bool wait_for(int64_t timeout_ms);
    bool done() const { return done_.load(std::memory_order_acquire); }
    bool has_exception() const { return done() && (!error_.empty()); }
    bool is_remote_exception() const { return done() && remote_exc_; }
    const std::string& payload() const { return payload_; }
    const std::string& error() const { return error_; }
    uint64_t request_id() const { return request_id_; }
    uint32_t slot_id() const { return slot_id_; }

    void fulfil(std::string&& payload, bool remote_exc);
    void fail(const std::string& why);

private:
    const uint64_t          request_id_;
    const uint32_t          slot_id_;
    std::mutex              mu_;
    std::condition_variable cv_;
    std::atomic<bool>       done_{false};
    bool                    remote_exc_ = false;
    std::string             payload_, error_;
};

struct InboundRequest {
    uint32_t    raw_tag = 0, base_tag = 0;
    uint64_t    request_id = 0;
    uint32_t    slot_id = 0;
    const char* payload_ptr = nullptr;  // borrowed from the receive slot; valid until the reply is posted
    size_t      payload_nbytes = 0;
};

using Writer = std::function<size_t(char* dst, size_t capacity)>;  // returns the bytes written

class RpcSession {
public:
    RpcSession(std::shared_ptr<Endpoint> endpoint, int local_send_handle, uintptr_t local_send_ptr, int local_recv_handle,
               uintptr_t local_recv_ptr, int remote_recv_handle, size_t slot_size, size_t slot_count,
               bool start_recv_pump = true);
    ~RpcSession();
    RpcSession(const RpcSession&)            = delete;
    RpcSession& operator=(const RpcSession&) = delete;

    std::shared_ptr<ClientFuture> call(uint32_t tag, const void* payload, size_t nbytes);
    std::shared_ptr<ClientFuture> call_inplace(uint32_t tag, const Writer& writer);
    // Blocks up to timeout_ms (< 0: until closed) for the next request.
    std::optional<InboundRequest> poll_request(int64_t timeout_ms = -1);
    void post_reply(uint32_t tag, uint64_t request_id, uint32_t client_slot_id, const void* payload, size_t nbytes);
    void post_reply_inplace(uint32_t tag, uint64_t request_id, uint32_t client_slot_id, const Writer& writer);
    void close();
    // The caller gave up on this request (timeout): a late reply only returns the slot.
    void detach_request(uint64_t request_id);

    size_t   slot_count() const { return slot_count_; }
    size_t   slot_size() const { return slot_size_; }
    size_t   payload_capacity() const { return slot_size_ - HEADER_SIZE; }
    bool     closed() const { return closed_.load(std::memory_order_acquire); }
    uint64_t requests_sent() const { return requests_sent_.load(); }
    uint64_t replies_received() const { return replies_received_.load(); }
    uint64_t requests_received() const { return requests_received_.load(); }

private:
    uint32_t acquire_slot();
    void     release_slot(uint32_t slot);
    void     post_committed(uint32_t tag, uint64_t request_id, uint32_t target_slot, size_t payload_bytes);
    void     settle_last_post();  // caller holds send_mu_: the write that last used the send buffer has completed
    void     recv_loop();
    bool     handle_arrival(uint32_t slot);  // false = malformed
    void     fail_all_pending(const std::string& why);

    std::shared_ptr<Endpoint> ep_;
    const int       send_h_, recv_h_, remote_recv_h_;
    const uintptr_t send_ptr_, recv_ptr_;
    const size_t    slot_size_, slot_count_;
    const bool      has_pump_;

    std::mutex send_mu_;  // one send buffer: header + payload are staged there, then written out
    std::shared_ptr<ReadWriteFuture> last_post_;  // under send_mu_: the write that still reads the send buffer
    std::mutex slot_mu_;
    std::condition_variable slot_cv_;
    std::deque<uint32_t>    free_slots_;

    std::mutex                                                  pending_mu_;
    std::unordered_map<uint64_t, std::shared_ptr<ClientFuture>> pending_;
    std::unordered_set<uint64_t>                                detached_;

    std::mutex                 inbox_mu_;
    std::condition_variable    inbox_cv_;
    std::deque<InboundRequest> inbox_;

    std::atomic<uint64_t> next_request_id_{1};
    std::atomic<bool>     closed_{false};
    std::atomic<uint64_t> requests_sent_{0}, replies_received_{0}, requests_received_{0};
    std::thread           pump_;
};

}  // namespace rpc
}  // namespace slime
