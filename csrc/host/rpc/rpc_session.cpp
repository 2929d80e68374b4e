#include "rpc/rpc_session.h"

#include <cstring>
#include <stdexcept>

#include "core/env.h"
#include "core/log.h"

namespace slime {
namespace rpc {

bool ClientFuture::wait_for(int64_t timeout_ms)
{
    std::unique_lock<std::mutex> g(mu_);
    auto ready = [&] { return done_.load(std::memory_order_acquire); };
    if (timeout_ms < 0) {
        cv_.wait(g, ready);
        return true;
    }
    return cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), ready);
}

void ClientFuture::fulfil(std::string&& payload, bool remote_exc)
{
    std::lock_guard<std::mutex> g(mu_);
    if (done_.load()) return;
    payload_    = std::move(payload);
    remote_exc_ = remote_exc;
    done_.store(true, std::memory_order_release);
    cv_.notify_all();
}

void ClientFuture::fail(const std::string& why)
{
    std::lock_guard<std::mutex> g(mu_);
    if (done_.load()) return;
    error_ = why.empty() ? "rpc session failed" : why;
    done_.store(true, std::memory_order_release);
    cv_.notify_all();
}

RpcSession::RpcSession(std::shared_ptr<Endpoint> endpoint, int local_send_handle, uintptr_t local_send_ptr,
                       int local_recv_handle, uintptr_t local_recv_ptr, int remote_recv_handle, size_t slot_size,
                       size_t slot_count, bool start_recv_pump):
    ep_(std::move(endpoint)), send_h_(local_send_handle), recv_h_(local_recv_handle), remote_recv_h_(remote_recv_handle),
    send_ptr_(local_send_ptr), recv_ptr_(local_recv_ptr), slot_size_(slot_size), slot_count_(slot_count),
    has_pump_(start_recv_pump)
{
    if (!ep_) throw std::invalid_argument("rpc session: endpoint is null");
    if (slot_size_ <= HEADER_SIZE) throw std::invalid_argument("rpc session: slot_size must exceed the 16-byte header");
    if (slot_count_ == 0 || slot_count_ > MAX_SLOT_COUNT) throw std::invalid_argument("rpc session: slot_count must be in [1, 65536]");
    for (uint32_t i = 0; i < slot_count_; ++i) free_slots_.push_back(i);
    if (has_pump_) pump_ = std::thread([this] { recv_loop(); });
}

RpcSession::~RpcSession()
{
    close();
}

uint32_t RpcSession::acquire_slot()
{
    std::unique_lock<std::mutex> g(slot_mu_);
    slot_cv_.wait(g, [&] { return closed_.load() || !free_slots_.empty(); });  // back-pressure: blocks while all slots are in flight
    if (closed_.load()) throw std::runtime_error("rpc session is closed");
    const uint32_t s = free_slots_.front();
    free_slots_.pop_front();
    return s;
}

void RpcSession::release_slot(uint32_t slot)
{
    {
        std::lock_guard<std::mutex> g(slot_mu_);
        free_slots_.push_back(slot);
    }
    slot_cv_.notify_one();
}

// The payload already sits behind the header position in the send buffer. Caller holds send_mu_.
void RpcSession::post_committed(uint32_t tag, uint64_t request_id, uint32_t target_slot, size_t payload_bytes)
{
    WireHeader h;
    h.tag        = tag;
    h.total_len  = static_cast<uint32_t>(HEADER_SIZE + payload_bytes);
    h.request_id = request_id;
    memcpy(reinterpret_cast<void*>(send_ptr_), &h, sizeof(h));
    std::vector<assign_tuple_t> assign{assign_tuple_t(static_cast<uintptr_t>(send_h_), static_cast<uintptr_t>(remote_recv_h_),
                                                      static_cast<uint64_t>(target_slot) * slot_size_, 0, h.total_len)};
    // The single send buffer may be reused as soon as this write has completed. Nobody waits for that here: the caller
    // goes on to wait for the reply (which cannot arrive before the request has), and whoever stages the next message
    // settles this write first (settle_last_post). That takes the write's acknowledgement off the path of a call.
    last_post_ = ep_->write_with_imm(assign, static_cast<int32_t>(target_slot));
}

void RpcSession::settle_last_post()
{
    if (!last_post_) return;
    auto fut = std::move(last_post_);
    last_post_.reset();
    // bounded like every other host wait: a peer that stops draining must not hold send_mu_ for ever
    static const int64_t post_ms = get_env<int64_t>("SLIME_RPC_POST_TIMEOUT_MS", 30000);
    const int32_t st = fut->wait(post_ms > 0 ? post_ms : 30000);
    if (st == TIME_OUT) throw std::runtime_error("rpc session: the previous write did not complete within " + std::to_string(post_ms) + " ms (status 402)");
    if (st != SUCCESS) throw std::runtime_error("rpc session: the previous write failed with status " + std::to_string(st));
}

std::shared_ptr<ClientFuture> RpcSession::call(uint32_t tag, const void* payload, size_t nbytes)
{
    return call_inplace(tag, [&](char* dst, size_t cap) -> size_t {
        if (nbytes > cap) throw std::length_error("rpc payload of " + std::to_string(nbytes) + " bytes exceeds the slot capacity of " + std::to_string(cap));
        if (nbytes) memcpy(dst, payload, nbytes);
        return nbytes;
    });
}

std::shared_ptr<ClientFuture> RpcSession::call_inplace(uint32_t tag, const Writer& writer)
{
    if (closed_.load()) throw std::runtime_error("rpc session is closed");
    const uint32_t slot = acquire_slot();
    const uint64_t rid  = next_request_id_.fetch_add(1);
    auto           fut  = std::make_shared<ClientFuture>(rid, slot);
    {
        std::lock_guard<std::mutex> g(pending_mu_);
        pending_[rid] = fut;  // registered before the request can possibly be answered
    }
    try {
        std::lock_guard<std::mutex> g(send_mu_);
        settle_last_post();
        const size_t n = writer(reinterpret_cast<char*>(send_ptr_) + HEADER_SIZE, payload_capacity());
        if (n > payload_capacity()) throw std::length_error("rpc writer produced more bytes than the slot holds");
        post_committed(tag & ~FLAG_MASK, rid, slot, n);
    }
    catch (...) {
        {
            std::lock_guard<std::mutex> g(pending_mu_);
            pending_.erase(rid);
        }
        release_slot(slot);
        throw;
    }
    requests_sent_.fetch_add(1);
    if (!has_pump_) {
        // single flight: drive the receive side here until our reply shows up
        while (!fut->done() && !closed_.load()) {
            auto rf = ep_->imm_recv();
            if (rf->wait(-1) != SUCCESS) {
                fail_all_pending("endpoint closed while waiting for a reply");
                break;
            }
            handle_arrival(static_cast<uint32_t>(rf->imm_data()) & 0xFFFF);
        }
    }
    return fut;
}

bool RpcSession::handle_arrival(uint32_t slot)
{
    if (slot >= slot_count_) {
        SLIME_LOG_ERROR("rpc session: immediate value names slot ", slot, " of ", slot_count_);
        return false;
    }
    const char* base = reinterpret_cast<const char*>(recv_ptr_) + static_cast<size_t>(slot) * slot_size_;
    WireHeader  h;
    memcpy(&h, base, sizeof(h));
    if (h.total_len < HEADER_SIZE || h.total_len > slot_size_) {
        SLIME_LOG_ERROR("rpc session: bad length ", h.total_len, " in slot ", slot);
        return false;
    }
    const size_t n = h.total_len - HEADER_SIZE;
    if (h.tag & REPLY_BIT) {
        std::shared_ptr<ClientFuture> fut;
        bool                          detached = false;
        {
            std::lock_guard<std::mutex> g(pending_mu_);
            auto it = pending_.find(h.request_id);
            if (it != pending_.end()) {
                fut = it->second;
                pending_.erase(it);
            }
            else if (detached_.erase(h.request_id) != 0) {
                detached = true;
            }
        }
        if (fut) {
            replies_received_.fetch_add(1);
            fut->fulfil(std::string(base + HEADER_SIZE, n), (h.tag & EXC_BIT) != 0);
            release_slot(slot);
        }
        else if (detached) {
            release_slot(slot);  // the late answer of an abandoned request only frees its slot
        }
        return true;
    }
    InboundRequest r;
    r.raw_tag        = h.tag;
    r.base_tag       = h.tag & ~FLAG_MASK;
    r.request_id     = h.request_id;
    r.slot_id        = slot;
    r.payload_ptr    = base + HEADER_SIZE;
    r.payload_nbytes = n;
    requests_received_.fetch_add(1);
    {
        std::lock_guard<std::mutex> g(inbox_mu_);
        inbox_.push_back(r);
    }
    inbox_cv_.notify_one();
    return true;
}

void RpcSession::recv_loop()
{
    while (!closed_.load()) {
        auto rf = ep_->imm_recv();
        const int32_t st = rf->wait(-1);
        if (closed_.load()) break;
        if (st != SUCCESS) {
            fail_all_pending("endpoint reported status " + std::to_string(st));
            break;
        }
        handle_arrival(static_cast<uint32_t>(rf->imm_data()) & 0xFFFF);
    }
    inbox_cv_.notify_all();
}

std::optional<InboundRequest> RpcSession::poll_request(int64_t timeout_ms)
{
    if (!has_pump_) {
        // no pump: take one arrival from the endpoint directly
        if (closed_.load()) return std::nullopt;
        auto rf = ep_->imm_recv();
        if (rf->wait(timeout_ms) != SUCCESS) return std::nullopt;
        handle_arrival(static_cast<uint32_t>(rf->imm_data()) & 0xFFFF);
    }
    std::unique_lock<std::mutex> g(inbox_mu_);
    auto ready = [&] { return closed_.load() || !inbox_.empty(); };
    if (timeout_ms < 0)
        inbox_cv_.wait(g, ready);
    else if (!inbox_cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), ready))
        return std::nullopt;
    if (inbox_.empty()) return std::nullopt;
    InboundRequest r = inbox_.front();
    inbox_.pop_front();
    return r;
}

void RpcSession::post_reply(uint32_t tag, uint64_t request_id, uint32_t client_slot_id, const void* payload, size_t nbytes)
{
    post_reply_inplace(tag, request_id, client_slot_id, [&](char* dst, size_t cap) -> size_t {
        if (nbytes > cap) throw std::length_error("rpc reply of " + std::to_string(nbytes) + " bytes exceeds the slot capacity of " + std::to_string(cap));
        if (nbytes) memcpy(dst, payload, nbytes);
        return nbytes;
    });
}

void RpcSession::post_reply_inplace(uint32_t tag, uint64_t request_id, uint32_t client_slot_id, const Writer& writer)
{
    if (closed_.load()) throw std::runtime_error("rpc session is closed");
    if (client_slot_id >= slot_count_) throw std::out_of_range("rpc reply names a slot outside the mailbox");
    std::lock_guard<std::mutex> g(send_mu_);
    settle_last_post();
    const size_t n = writer(reinterpret_cast<char*>(send_ptr_) + HEADER_SIZE, payload_capacity());
    if (n > payload_capacity()) throw std::length_error("rpc writer produced more bytes than the slot holds");
    post_committed(tag | REPLY_BIT, request_id, client_slot_id, n);
}

void RpcSession::detach_request(uint64_t request_id)
{
    std::lock_guard<std::mutex> g(pending_mu_);
    if (pending_.erase(request_id) != 0) detached_.insert(request_id);
}

void RpcSession::fail_all_pending(const std::string& why)
{
    std::unordered_map<uint64_t, std::shared_ptr<ClientFuture>> victims;
    {
        std::lock_guard<std::mutex> g(pending_mu_);
        victims.swap(pending_);
    }
    for (auto& kv : victims) kv.second->fail(why);
}

void RpcSession::close()
{
    if (closed_.exchange(true)) return;
    fail_all_pending("rpc session closed");
    slot_cv_.notify_all();
    inbox_cv_.notify_all();
    if (ep_) ep_->cancel_all();  // wakes the pump out of its immediate receive
    if (pump_.joinable()) pump_.join();
}

}  // namespace rpc
}  // namespace slime
