#include "transport/tcp_endpoint.h"

#include <arpa/inet.h>
#include <cerrno>
#include <cstring>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/uio.h>
#include <sys/types.h>
#include <unistd.h>

#include "core/env.h"
#include "core/log.h"
#include "obs/obs.h"

namespace slime {

namespace {

constexpr uint32_t kMagic = 0x534c494dU;  // "SLIM"
enum Kind : uint8_t { REQ_WRITE = 1, REQ_READ = 2, REQ_SEND = 3, RSP_ACK = 4, RSP_DATA = 5 };
enum Flags : uint8_t { F_LAST = 1, F_IMM = 2 };

#pragma pack(push, 1)
struct WireHdr {
    uint32_t magic  = kMagic;
    uint8_t  kind   = 0;
    uint8_t  flags  = 0;
    uint16_t rsvd   = 0;
    uint64_t id     = 0;
    uint64_t handle = 0;
    uint64_t offset = 0;
    uint64_t length = 0;
    int32_t  imm    = 0;  // immediate data, or the piece index of a read
    int32_t  status = 0;
};
#pragma pack(pop)
static_assert(sizeof(WireHdr) == 48, "wire header is 48 bytes");

bool send_all(int fd, const void* buf, size_t n)
{
    const char* p = static_cast<const char*>(buf);
    while (n > 0) {
        ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
        if (w < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        if (w == 0) return false;
        p += w;
        n -= static_cast<size_t>(w);
    }
    return true;
}

// Header and payload in one system call (one segment on the wire for small payloads instead of two).
bool send_hdr_and_payload(int fd, const void* hdr, size_t hdr_len, const void* payload, size_t n)
{
    if (n == 0) return send_all(fd, hdr, hdr_len);
    iovec  iov[2] = {{const_cast<void*>(hdr), hdr_len}, {const_cast<void*>(payload), n}};
    msghdr m{};
    m.msg_iov    = iov;
    m.msg_iovlen = 2;
    ssize_t w;
    do {
        w = ::sendmsg(fd, &m, MSG_NOSIGNAL);
    } while (w < 0 && errno == EINTR);
    if (w <= 0) return false;
    size_t done = static_cast<size_t>(w);
    if (done < hdr_len) {  // rare: finish the header, then the payload
        if (!send_all(fd, static_cast<const char*>(hdr) + done, hdr_len - done)) return false;
        done = hdr_len;
    }
    const size_t sent = done - hdr_len;
    return sent >= n || send_all(fd, static_cast<const char*>(payload) + sent, n - sent);
}

bool recv_all(int fd, void* buf, size_t n)
{
    char* p = static_cast<char*>(buf);
    while (n > 0) {
        ssize_t r = ::recv(fd, p, n, 0);
        if (r < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        if (r == 0) return false;
        p += r;
        n -= static_cast<size_t>(r);
    }
    return true;
}

bool drain(int fd, uint64_t n)
{
    char scratch[65536];
    while (n > 0) {
        const size_t k = static_cast<size_t>(std::min<uint64_t>(n, sizeof(scratch)));
        if (!recv_all(fd, scratch, k)) return false;
        n -= k;
    }
    return true;
}

void tune(int fd)
{
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    int buf = 4 << 20;
    setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
    setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
}

}  // namespace

TcpEndpoint::TcpEndpoint(const std::string& bind_host, int port, int /*num_lanes*/): host_(bind_host)
{
    listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
    if (listen_fd_ < 0) SLIME_FAIL("tcp endpoint: socket() failed: ", strerror(errno));
    int one = 1;
    setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port   = htons(static_cast<uint16_t>(port));
    if (inet_pton(AF_INET, bind_host.c_str(), &addr.sin_addr) != 1) addr.sin_addr.s_addr = htonl(INADDR_ANY);
    if (::bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(listen_fd_, 64) != 0) {
        const std::string why = strerror(errno);
        ::close(listen_fd_);
        listen_fd_ = -1;
        SLIME_FAIL("tcp endpoint: bind/listen on ", bind_host, ":", port, " failed: ", why);
    }
    socklen_t len = sizeof(addr);
    getsockname(listen_fd_, reinterpret_cast<sockaddr*>(&addr), &len);
    port_     = ntohs(addr.sin_port);
    obs_link_ = obs::register_link("tcp:" + host_ + ":" + std::to_string(port_), "tcp");
    acceptor_ = std::thread([this] { acceptor_loop(); });
}

TcpEndpoint::~TcpEndpoint()
{
    shutdown();
}

Json TcpEndpoint::endpoint_info()
{
    Json j       = Json::object();
    j["kind"]    = "tcp";
    j["host"]    = host_;
    j["port"]    = port_;
    j["mr_info"] = mr_info();
    return j;
}

int TcpEndpoint::connect(const Json& remote_info)
{
    if (connected_.load()) return 0;
    // remote regions: keep the owner's handle as the transport key
    std::vector<std::pair<int64_t, std::string>> order;
    for (const auto& kv : remote_info["mr_info"].fields()) order.emplace_back(kv.second["handle"].as_int(), kv.first);
    std::sort(order.begin(), order.end());
    for (const auto& e : order) register_remote_memory_region(e.second, remote_info["mr_info"][e.second]);

    const std::string host = remote_info["host"].string_or("127.0.0.1");
    const int         port = static_cast<int>(remote_info["port"].as_int());
    addrinfo          hints{}, *res = nullptr;
    hints.ai_family   = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    if (getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res) != 0 || res == nullptr)
        SLIME_FAIL("tcp endpoint: cannot resolve ", host);
    int fd = -1;
    for (int attempt = 0; attempt < 50 && fd < 0; ++attempt) {
        fd = ::socket(AF_INET, SOCK_STREAM, 0);
        if (fd >= 0 && ::connect(fd, res->ai_addr, res->ai_addrlen) != 0) {
            ::close(fd);
            fd = -1;
            usleep(20000);
        }
    }
    freeaddrinfo(res);
    if (fd < 0) SLIME_FAIL("tcp endpoint: cannot connect to ", host, ":", port);
    tune(fd);
    out_fd_ = fd;
    connected_.store(true);
    sender_   = std::thread([this] { sender_loop(); });
    receiver_ = std::thread([this] { receiver_loop(); });
    return 0;
}

// ------------------------------------------------------------------------------------------------
// submission
// ------------------------------------------------------------------------------------------------
std::shared_ptr<ReadWriteFuture> TcpEndpoint::submit_one_sided(OpCode opcode, const std::vector<assign_tuple_t>& assign, int32_t imm,
                                                               void* stream)
{
    auto st = make_op_state(1, opcode);
    // with stream-ordered signals the sender thread posts only once the stream has reached this point
    if (stream != nullptr && !engine_env().bypass_device_signal) st->signal->bind_stream(stream);
    st->signal->record_gpu_ready();
    uint64_t bytes = 0;
    for (const auto& a : assign) bytes += std::get<4>(a);
    st->bytes   = bytes;
    st->link_id = obs_link_;
    obs::record_submit(obs_link_, obs::op_index(opcode), assign.size(), bytes);
    auto fut = std::make_shared<ReadWriteFuture>(st);
    if (!connected_.load() || stopping_.load() || broken_.load()) {
        complete(st, FAILED);
        return fut;
    }
    Op op;
    op.opcode = opcode;
    op.assign = assign;
    op.imm    = imm;
    op.state  = st;
    op.id     = next_id_.fetch_add(1);
    // a read posts only headers; a write is posted by the caller only when it is small enough not to hold the caller up
    if (!try_post_inline(op, opcode == OpCode::READ ? 0 : bytes)) enqueue(std::move(op));
    return fut;
}

void TcpEndpoint::enqueue(Op&& op)
{
    {
        std::lock_guard<std::mutex> g(submit_mu_);
        submit_q_.push_back(std::move(op));
    }
    submit_cv_.notify_one();
}

bool TcpEndpoint::try_post_inline(Op& op, uint64_t bytes)
{
    constexpr uint64_t kInlineBytes = 256 * 1024;
    if (bytes > kInlineBytes || !op.state->signal->is_gpu_ready()) return false;
    if (op.opcode == OpCode::READ && op.assign.empty()) return false;  // completed by the sender loop without a post
    {
        std::lock_guard<std::mutex> g(submit_mu_);
        if (posting_ || !submit_q_.empty() || stopping_.load()) return false;
        posting_ = true;  // from here on every other operation queues up behind this one
    }
    {
        std::lock_guard<std::mutex> g(inflight_mu_);
        inflight_[op.id] = op;
    }
    const bool ok = post_op(op);
    {
        std::lock_guard<std::mutex> g(submit_mu_);
        posting_ = false;
    }
    submit_cv_.notify_one();  // the sender thread may have been waiting for its turn
    if (!ok) {
        obs::record_post_failure(obs_link_, obs::op_index(op.opcode));
        broken_.store(true);
        fail_everything(FAILED);
    }
    else if (broken_.load()) {
        fail_everything(FAILED);  // the link died while this operation was on its way: nobody will answer it
    }
    return true;
}

std::shared_ptr<ReadWriteFuture> TcpEndpoint::read(const std::vector<assign_tuple_t>& assign, void* stream)
{
    return submit_one_sided(OpCode::READ, assign, 0, stream);
}
std::shared_ptr<ReadWriteFuture> TcpEndpoint::write(const std::vector<assign_tuple_t>& assign, void* stream)
{
    return submit_one_sided(OpCode::WRITE, assign, 0, stream);
}
std::shared_ptr<ReadWriteFuture> TcpEndpoint::write_with_imm(const std::vector<assign_tuple_t>& assign, int32_t imm, void* stream)
{
    return submit_one_sided(OpCode::WRITE_WITH_IMM, assign, imm, stream);
}

std::shared_ptr<ImmRecvFuture> TcpEndpoint::imm_recv(void*)
{
    auto st = make_op_state(1, OpCode::RECV);
    if (engine_env().with_time_trace) st->trace_start_ns.store(monotonic_ns());
    auto fut = std::make_shared<ImmRecvFuture>(st);
    std::unique_lock<std::mutex> g(imm_mu_);
    if (!imm_events_.empty()) {
        const int32_t v = imm_events_.front();
        imm_events_.pop_front();
        g.unlock();
        st->imm_data.store(v);
        st->trace_end_ns.store(monotonic_ns());
        st->signal->set_comm_done(0);
        return fut;
    }
    if (shut_.load()) {
        g.unlock();
        st->fail(FAILED);
        st->signal->set_comm_done(0);
        return fut;
    }
    imm_waiters_.push_back(st);
    return fut;
}

std::shared_ptr<SendFuture> TcpEndpoint::send(const chunk_tuple_t& chunk, void* stream)
{
    auto st  = make_op_state(1, OpCode::SEND);
    auto fut = std::make_shared<SendFuture>(st);
    if (stream != nullptr && !engine_env().bypass_device_signal) st->signal->bind_stream(stream);
    st->signal->record_gpu_ready();
    if (!connected_.load() || stopping_.load() || broken_.load()) {
        complete(st, FAILED);
        return fut;
    }
    Op op;
    op.opcode = OpCode::SEND;
    op.chunk  = chunk;
    op.state  = st;
    op.id     = next_id_.fetch_add(1);
    if (!try_post_inline(op, std::get<2>(chunk))) enqueue(std::move(op));
    return fut;
}

std::shared_ptr<RecvFuture> TcpEndpoint::recv(const chunk_tuple_t& chunk, void*)
{
    auto st  = make_op_state(1, OpCode::RECV);
    auto fut = std::make_shared<RecvFuture>(st);
    const uintptr_t ptr = std::get<0>(chunk) + std::get<1>(chunk);
    const size_t    len = std::get<2>(chunk);
    std::unique_lock<std::mutex> g(msg_mu_);
    if (!msg_unexpected_.empty()) {
        std::vector<uint8_t> m = std::move(msg_unexpected_.front());
        msg_unexpected_.pop_front();
        g.unlock();
        memcpy(reinterpret_cast<void*>(ptr), m.data(), std::min(len, m.size()));
        if (m.size() > len) st->fail(ASSIGNMENT_BATCH_OVERFLOW);
        st->signal->set_comm_done(0);
        return fut;
    }
    if (shut_.load()) {
        g.unlock();
        st->fail(FAILED);
        st->signal->set_comm_done(0);
        return fut;
    }
    recv_posted_.push_back(PendingRecv{ptr, len, st});
    return fut;
}

// ------------------------------------------------------------------------------------------------
// client side threads
// ------------------------------------------------------------------------------------------------
bool TcpEndpoint::post_op(Op& op)
{
    if (fault_reset_.load() > 0) {
        fault_reset_.fetch_sub(1);
        ::shutdown(out_fd_, SHUT_RDWR);
        return false;
    }
    const obs::OpIndex oi = obs::op_index(op.opcode);
    if (op.opcode == OpCode::SEND) {
        WireHdr h;
        h.kind   = REQ_SEND;
        h.flags  = F_LAST;
        h.id     = op.id;
        h.length = std::get<2>(op.chunk);
        return send_hdr_and_payload(out_fd_, &h, sizeof(h), reinterpret_cast<const void*>(std::get<0>(op.chunk) + std::get<1>(op.chunk)), h.length);
    }
    // Every piece is checked before the first byte leaves: a batch with a piece that names an unknown region or runs
    // past one fails as a whole, moves nothing, and leaves nothing in flight for the peer to answer.
    std::vector<MemoryRegion> locals(op.assign.size()), remotes(op.assign.size());
    for (size_t i = 0; i < op.assign.size(); ++i) {
        const auto& a = op.assign[i];
        if (!local_pool_->get_mr(static_cast<int32_t>(std::get<0>(a)), locals[i])
            || !remote_pool_->get_remote_mr(static_cast<int32_t>(std::get<1>(a)), remotes[i])
            || !locals[i].contains(std::get<3>(a), std::get<4>(a)) || !remotes[i].contains(std::get<2>(a), std::get<4>(a))) {
            SLIME_LOG_ERROR("tcp endpoint: assignment ", i, " names an unknown region or exceeds it");
            {
                std::lock_guard<std::mutex> g(inflight_mu_);
                inflight_.erase(op.id);
            }
            complete(op.state, FAILED);
            return true;
        }
    }
    uint64_t posted = 0;
    for (size_t i = 0; i < op.assign.size(); ++i) {
        const auto&         a      = op.assign[i];
        const MemoryRegion& local  = locals[i];
        const MemoryRegion& remote = remotes[i];
        const bool last = i + 1 == op.assign.size();
        WireHdr    h;
        h.id     = op.id;
        h.handle = remote.rkey;  // the owner's handle
        h.offset = std::get<2>(a);
        h.length = std::get<4>(a);
        if (op.opcode == OpCode::READ) {
            h.kind = REQ_READ;
            h.imm  = static_cast<int32_t>(i);
            if (!send_all(out_fd_, &h, sizeof(h))) return false;
        }
        else {
            h.kind  = REQ_WRITE;
            h.flags = last ? F_LAST : 0;
            if (last && op.opcode == OpCode::WRITE_WITH_IMM) {
                h.flags |= F_IMM;
                h.imm = op.imm;
            }
            if (!send_hdr_and_payload(out_fd_, &h, sizeof(h), reinterpret_cast<const void*>(local.addr + std::get<3>(a)), h.length)) return false;
        }
        posted += h.length;
    }
    if (op.assign.empty() && op.opcode != OpCode::READ) {
        WireHdr h;
        h.kind   = REQ_WRITE;
        h.flags  = F_LAST | (op.opcode == OpCode::WRITE_WITH_IMM ? F_IMM : 0);
        h.id     = op.id;
        h.handle = ~0ull;
        h.imm    = op.imm;
        if (!send_all(out_fd_, &h, sizeof(h))) return false;
    }
    obs::record_post_batch(obs_link_, oi, op.assign.size(), posted);
    return true;
}

void TcpEndpoint::sender_loop()
{
    while (true) {
        Op op;
        {
            std::unique_lock<std::mutex> g(submit_mu_);
            submit_cv_.wait(g, [&] { return stopping_.load() || (!submit_q_.empty() && !posting_); });
            if (stopping_.load()) return;
            op = std::move(submit_q_.front());
            submit_q_.pop_front();
            posting_ = true;
        }
        struct Turn {  // hands the turn back however this iteration ends
            TcpEndpoint* e;
            ~Turn()
            {
                {
                    std::lock_guard<std::mutex> g(e->submit_mu_);
                    e->posting_ = false;
                }
                e->submit_cv_.notify_one();
            }
        } turn{this};
        // head of line: operations leave in submission order, so a buffer that is not ready yet holds back what follows
        while (!op.state->signal->is_gpu_ready() && !stopping_.load()) std::this_thread::sleep_for(std::chrono::microseconds(20));
        if (stopping_.load()) {
            complete(op.state, FAILED);
            return;
        }
        if (op.opcode == OpCode::READ && op.assign.empty()) {
            complete(op.state, SUCCESS);
            continue;
        }
        {
            std::lock_guard<std::mutex> g(inflight_mu_);
            inflight_[op.id] = op;
        }
        if (!post_op(op)) {
            obs::record_post_failure(obs_link_, obs::op_index(op.opcode));
            broken_.store(true);
            fail_everything(FAILED);
            return;
        }
        if (broken_.load()) {  // the link died while this operation was on its way: nobody will answer it
            fail_everything(FAILED);
            return;
        }
    }
}

void TcpEndpoint::receiver_loop()
{
    // per-read bookkeeping: pieces still missing
    std::unordered_map<uint64_t, size_t> read_left;
    while (!stopping_.load()) {
        WireHdr h;
        if (!recv_all(out_fd_, &h, sizeof(h)) || h.magic != kMagic) break;
        if (h.kind == RSP_ACK) {
            if (fault_drop_ack_.load() > 0) {
                fault_drop_ack_.fetch_sub(1);
                continue;
            }
            Op op;
            {
                std::lock_guard<std::mutex> g(inflight_mu_);
                auto it = inflight_.find(h.id);
                if (it == inflight_.end()) continue;
                op = std::move(it->second);
                inflight_.erase(it);
            }
            complete(op.state, h.status);
        }
        else if (h.kind == RSP_DATA) {
            std::shared_ptr<EndpointOpState> st;
            assign_tuple_t                   a{};
            size_t                           n_pieces = 0;
            {
                std::lock_guard<std::mutex> g(inflight_mu_);
                auto it = inflight_.find(h.id);
                if (it != inflight_.end() && static_cast<size_t>(h.imm) < it->second.assign.size()) {
                    st       = it->second.state;
                    a        = it->second.assign[h.imm];
                    n_pieces = it->second.assign.size();
                }
            }
            MemoryRegion local;
            const bool   ok = st && h.status == SUCCESS && local_pool_->get_mr(static_cast<int32_t>(std::get<0>(a)), local)
                            && local.contains(std::get<3>(a), h.length);
            if (ok) {
                if (!recv_all(out_fd_, reinterpret_cast<void*>(local.addr + std::get<3>(a)), h.length)) break;
            }
            else {
                if (!drain(out_fd_, h.length)) break;
                if (st) st->fail(h.status != SUCCESS ? h.status : FAILED);
            }
            if (!st) continue;
            auto it = read_left.find(h.id);
            if (it == read_left.end()) it = read_left.emplace(h.id, n_pieces).first;
            if (--it->second == 0) {
                read_left.erase(it);
                {
                    std::lock_guard<std::mutex> g(inflight_mu_);
                    inflight_.erase(h.id);
                }
                complete(st, st->completion_status.load());
            }
        }
    }
    if (!stopping_.load()) {
        broken_.store(true);  // the peer is gone: whatever is submitted from now on fails at once
        fail_everything(FAILED);
    }
}

// ------------------------------------------------------------------------------------------------
// server side
// ------------------------------------------------------------------------------------------------
void TcpEndpoint::acceptor_loop()
{
    while (!stopping_.load()) {
        pollfd p{listen_fd_, POLLIN, 0};
        const int r = ::poll(&p, 1, 200);
        if (r <= 0) continue;
        const int fd = ::accept(listen_fd_, nullptr, nullptr);
        if (fd < 0) continue;
        tune(fd);
        std::lock_guard<std::mutex> g(servers_mu_);
        if (stopping_.load()) {
            ::close(fd);
            return;
        }
        server_fds_.push_back(fd);
        servers_.emplace_back([this, fd] { server_loop(fd); });
    }
}

void TcpEndpoint::server_loop(int fd)
{
    int32_t batch_status = SUCCESS;  // first failure inside the current write batch
    while (!stopping_.load()) {
        WireHdr h;
        if (!recv_all(fd, &h, sizeof(h)) || h.magic != kMagic) break;
        if (h.kind == REQ_WRITE) {
            MemoryRegion r;
            bool         ok = true;
            if (h.length > 0 || h.handle != ~0ull) {
                ok = local_pool_->get_mr(static_cast<int32_t>(h.handle), r) && r.contains(h.offset, h.length);
                if (ok && fault_fail_write_.load() > 0) {
                    fault_fail_write_.fetch_sub(1);
                    ok = false;
                }
                if (ok) {
                    if (!recv_all(fd, reinterpret_cast<void*>(r.addr + h.offset), h.length)) break;
                }
                else {
                    if (!drain(fd, h.length)) break;
                    if (h.handle != ~0ull || h.length > 0) batch_status = FAILED;
                }
            }
            if (h.flags & F_LAST) {
                if ((h.flags & F_IMM) && batch_status == SUCCESS) deliver_imm(h.imm);
                WireHdr ack;
                ack.kind   = RSP_ACK;
                ack.id     = h.id;
                ack.status = batch_status;
                batch_status = SUCCESS;
                if (!send_all(fd, &ack, sizeof(ack))) break;
            }
        }
        else if (h.kind == REQ_READ) {
            MemoryRegion r;
            const bool   ok = local_pool_->get_mr(static_cast<int32_t>(h.handle), r) && r.contains(h.offset, h.length);
            WireHdr      rsp;
            rsp.kind   = RSP_DATA;
            rsp.id     = h.id;
            rsp.imm    = h.imm;
            rsp.status = ok ? SUCCESS : FAILED;
            rsp.length = ok ? h.length : 0;
            if (!send_hdr_and_payload(fd, &rsp, sizeof(rsp), reinterpret_cast<const void*>(r.addr + h.offset), ok ? h.length : 0)) break;
        }
        else if (h.kind == REQ_SEND) {
            // The length comes from the peer: a corrupt or hostile header must neither pin gigabytes of host memory
            // nor take the process down with an allocation failure inside this thread. Above the limit
            // (SLIME_TCP_MAX_MESSAGE_BYTES, default 1 GiB) the connection is closed.
            static const uint64_t max_msg = get_env<uint64_t>("SLIME_TCP_MAX_MESSAGE_BYTES", 1ull << 30);
            if (h.length > max_msg) {
                SLIME_LOG_WARN("tcp endpoint: message of ", h.length, " bytes exceeds the limit of ", max_msg, "; closing the connection");
                break;
            }
            std::vector<uint8_t> payload;
            try {
                payload.resize(h.length);
            }
            catch (const std::exception&) {
                SLIME_LOG_WARN("tcp endpoint: no memory for a message of ", h.length, " bytes; closing the connection");
                break;
            }
            if (h.length && !recv_all(fd, payload.data(), h.length)) break;
            deliver_message(std::move(payload));
            WireHdr ack;
            ack.kind = RSP_ACK;
            ack.id   = h.id;
            if (!send_all(fd, &ack, sizeof(ack))) break;
        }
        else {
            break;
        }
    }
}

void TcpEndpoint::deliver_imm(int32_t imm)
{
    std::shared_ptr<EndpointOpState> st;
    {
        std::lock_guard<std::mutex> g(imm_mu_);
        if (imm_waiters_.empty()) {
            imm_events_.push_back(imm);
            return;
        }
        st = imm_waiters_.front();
        imm_waiters_.pop_front();
    }
    st->imm_data.store(imm);
    st->trace_end_ns.store(monotonic_ns());
    st->signal->set_comm_done(0);
}

void TcpEndpoint::deliver_message(std::vector<uint8_t>&& payload)
{
    PendingRecv pr{};
    {
        std::lock_guard<std::mutex> g(msg_mu_);
        if (recv_posted_.empty()) {
            msg_unexpected_.push_back(std::move(payload));
            return;
        }
        pr = recv_posted_.front();
        recv_posted_.pop_front();
    }
    memcpy(reinterpret_cast<void*>(pr.ptr), payload.data(), std::min(pr.length, payload.size()));
    if (payload.size() > pr.length) pr.state->fail(ASSIGNMENT_BATCH_OVERFLOW);
    pr.state->signal->set_comm_done(0);
}

// ------------------------------------------------------------------------------------------------
// completion / teardown
// ------------------------------------------------------------------------------------------------
void TcpEndpoint::complete(const std::shared_ptr<EndpointOpState>& st, int32_t status)
{
    if (status != SUCCESS) st->fail(status);
    if (!st->obs_completed.exchange(true)) {
        const obs::OpIndex oi = obs::op_index(st->opcode);
        if (st->opcode == OpCode::READ || st->opcode == OpCode::WRITE || st->opcode == OpCode::WRITE_WITH_IMM) {
            if (st->completion_status.load() == SUCCESS)
                obs::record_complete(st->link_id, oi, st->bytes);
            else
                obs::record_fail(st->link_id, oi, st->bytes);
        }
    }
    st->signal->set_comm_done(0);
}

void TcpEndpoint::fail_everything(int32_t status)
{
    std::vector<std::shared_ptr<EndpointOpState>> victims;
    {
        std::lock_guard<std::mutex> g(submit_mu_);
        for (auto& op : submit_q_) victims.push_back(op.state);
        submit_q_.clear();
    }
    {
        std::lock_guard<std::mutex> g(inflight_mu_);
        for (auto& kv : inflight_) victims.push_back(kv.second.state);
        inflight_.clear();
    }
    for (auto& st : victims) complete(st, status);
    std::deque<std::shared_ptr<EndpointOpState>> waiters;
    {
        std::lock_guard<std::mutex> g(imm_mu_);
        waiters.swap(imm_waiters_);
    }
    for (auto& st : waiters) {
        st->fail(status);
        st->signal->set_comm_done(0);
    }
    std::deque<PendingRecv> recvs;
    {
        std::lock_guard<std::mutex> g(msg_mu_);
        recvs.swap(recv_posted_);
    }
    for (auto& r : recvs) {
        r.state->fail(status);
        r.state->signal->set_comm_done(0);
    }
}

void TcpEndpoint::cancel_all()
{
    fail_everything(FAILED);
}

void TcpEndpoint::shutdown()
{
    if (shut_.exchange(true)) return;
    stopping_.store(true);
    submit_cv_.notify_all();
    if (out_fd_ >= 0) ::shutdown(out_fd_, SHUT_RDWR);
    if (listen_fd_ >= 0) ::shutdown(listen_fd_, SHUT_RDWR);
    {
        std::lock_guard<std::mutex> g(servers_mu_);
        for (int fd : server_fds_) ::shutdown(fd, SHUT_RDWR);
    }
    if (sender_.joinable()) sender_.join();
    if (receiver_.joinable()) receiver_.join();
    if (acceptor_.joinable()) acceptor_.join();
    std::vector<std::thread> servers;
    {
        std::lock_guard<std::mutex> g(servers_mu_);
        servers.swap(servers_);
    }
    for (auto& t : servers)
        if (t.joinable()) t.join();
    fail_everything(FAILED);
    if (out_fd_ >= 0) ::close(out_fd_);
    if (listen_fd_ >= 0) ::close(listen_fd_);
    for (int fd : server_fds_) ::close(fd);
    out_fd_ = listen_fd_ = -1;
    server_fds_.clear();
    connected_.store(false);
}

void TcpEndpoint::inject_fault(const std::string& what, int count)
{
    if (what == "drop_ack") fault_drop_ack_.store(count);
    else if (what == "reset") fault_reset_.store(count);
    else if (what == "fail_write") fault_fail_write_.store(count);
    else SLIME_FAIL("unknown fault '", what, "'");
}

}  // namespace slime
