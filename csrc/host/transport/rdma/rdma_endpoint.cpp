#include "transport/rdma/rdma_endpoint.h"

#include <algorithm>
#include <cstring>
#include <random>
#include <stdexcept>

#include "core/env.h"
#include "core/log.h"
#include "obs/obs.h"
#include "transport/rdma/rdma_worker.h"

namespace slime {
namespace rdma {

namespace {
constexpr int      kSignalEvery = 32;
constexpr uint32_t kTxSlots     = 8192;
constexpr uint32_t kOverflowBit = 0x80000000u;

uint32_t random_psn()
{
    static std::mt19937       gen{std::random_device{}()};
    static std::mutex         mu;
    std::lock_guard<std::mutex> g(mu);
    return gen() & 0xffffff;
}
}  // namespace

std::shared_ptr<RdmaEndpoint> RdmaEndpoint::create(const std::string& device, int port, const std::string& link_type, int num_qp)
{
    return create(ContextManager::get().acquire(device, port, link_type), num_qp, nullptr);
}

std::shared_ptr<RdmaEndpoint> RdmaEndpoint::create(std::shared_ptr<RdmaContext> ctx, int num_qp, std::shared_ptr<RdmaWorker> worker)
{
    if (!ctx) throw std::runtime_error("RDMA endpoint needs a context");
    if (num_qp <= 0) num_qp = engine_env().qp_num;
    if (num_qp < 1 || num_qp > 32) throw std::runtime_error("num_qp must be in [1, 32]");
    std::shared_ptr<RdmaEndpoint> ep(new RdmaEndpoint(ctx, num_qp));
    for (auto& ch : ep->ch_)
        for (auto& l : ch.lanes) ctx->add_sink(l.qpn, ep);
    ep->worker_ = worker ? std::move(worker) : RdmaWorker::for_node(ctx->numa_node());
    ep->worker_->add(ep);
    return ep;
}

void RdmaEndpoint::set_worker(std::shared_ptr<RdmaWorker> worker)
{
    if (shut_.load()) return;
    if (!worker) worker = RdmaWorker::for_node(ctx_->numa_node());
    if (worker == worker_) return;
    // joined to the new worker before leaving the old one: process() serialises itself, so a moment with two
    // workers is harmless, a moment with none would stall queued work
    auto old = worker_;
    worker->add(shared_from_this());
    worker_ = worker;
    if (old) old->remove(this);
    worker_->wake();
}

RdmaEndpoint::RdmaEndpoint(std::shared_ptr<RdmaContext> ctx, int num_qp):
    ctx_(std::move(ctx)), num_qp_(num_qp), tx_slots_(kTxSlots), free_slots_(kTxSlots)
{
    local_pool_       = ctx_->shared_pool();
    own_pool_         = local_pool_;
    stripe_min_bytes_ = get_env<uint64_t>("SLIME_STRIPE_MIN_BYTES", 64 << 10);
    for (uint32_t i = 0; i < kTxSlots; ++i) free_slots_.try_push(i);

    const EngineEnv& env = engine_env();
    int send_wr = env.max_send_wr;
    if (ctx_->max_qp_wr() > 0) send_wr = std::min(send_wr, ctx_->max_qp_wr());
    QpCaps io{send_wr, std::min(env.max_io_fifo_depth, std::max(1, ctx_->max_qp_wr())), 0};
    QpCaps msg{send_wr, std::min(env.max_msg_fifo_depth, std::max(1, ctx_->max_qp_wr())), 0};
    meta_depth_ = std::min(env.max_msg_fifo_depth, std::max(1, ctx_->max_qp_wr()));
    QpCaps meta{meta_depth_, meta_depth_, static_cast<int>(sizeof(MetaMsg))};
    init_channel(ch_[CH_IO], num_qp_, io);
    init_channel(ch_[CH_MSG], num_qp_, msg);
    init_channel(ch_[CH_META], 1, meta);
    ch_[CH_IO].recv_window   = io.max_recv_wr;
    ch_[CH_MSG].recv_window  = msg.max_recv_wr;
    ch_[CH_META].recv_window = meta_depth_;

    static_assert(sizeof(MetaMsg) == 64, "meta message is one cache line");
    meta_buf_.assign(static_cast<size_t>(meta_depth_) * sizeof(MetaMsg), 0);
    meta_name_      = "sys.meta." + std::to_string(ch_[CH_META].lanes[0].qpn);
    const int32_t h = own_pool_->register_memory_region(reinterpret_cast<uintptr_t>(meta_buf_.data()), meta_buf_.size(), meta_name_);
    own_pool_->get_mr(h, meta_mr_);
}

RdmaEndpoint::~RdmaEndpoint()
{
    shutdown();
}

void RdmaEndpoint::init_channel(Channel& ch, int lanes, const QpCaps& caps)
{
    ch.lanes.reserve(lanes);
    for (int i = 0; i < lanes; ++i) {
        Lane l;
        l.qp = ctx_->dev().create_qp(ctx_->pd(), ctx_->cq(), caps, l.qpn);
        if (!l.qp) throw std::runtime_error("cannot create a queue pair on " + ctx_->device_name());
        if (ctx_->dev().qp_to_init(l.qp, ctx_->port()) != 0) throw std::runtime_error("queue pair INIT transition failed");
        l.psn = random_psn();
        l.credits.store(caps.max_send_wr);
        ch.lanes.push_back(std::move(l));
    }
}

Json RdmaEndpoint::endpoint_info()
{
    Json j         = Json::object();
    j["kind"]      = "rdma";
    j["device"]    = ctx_->device_name();
    j["port"]      = ctx_->port();
    j["link_type"] = ctx_->is_roce() ? "RoCE" : "IB";
    const char* names[3] = {"io", "msg", "meta"};
    for (int c = 0; c < 3; ++c) {
        Json arr = Json::array();
        for (auto& l : ch_[c].lanes) {
            QpInfo q;
            q.qpn  = l.qpn;
            q.psn  = l.psn;
            q.gid  = ctx_->gid();
            q.gidx = ctx_->gid_index();
            q.lid  = ctx_->lid();
            q.mtu  = ctx_->mtu();
            arr.push_back(q.to_json());
        }
        j[names[c]] = arr;
    }
    j["mr_info"] = mr_info();
    return j;
}

int RdmaEndpoint::connect_channel(Channel& ch, const Json& remote, const char* name)
{
    if (!remote.is_array() || remote.size() != ch.lanes.size()) {
        SLIME_LOG_ERROR("peer has ", remote.is_array() ? remote.size() : 0, " queue pairs in channel ", name, ", this side has ", ch.lanes.size());
        return -1;
    }
    const EngineEnv& env = engine_env();
    for (size_t i = 0; i < ch.lanes.size(); ++i) {
        const QpInfo peer = QpInfo::from_json(remote[i]);
        QpRoute      r;
        r.dest_qpn           = peer.qpn;
        r.dest_psn           = peer.psn;
        r.local_psn          = ch.lanes[i].psn;
        r.mtu                = std::min(ctx_->mtu(), peer.mtu);
        r.dest_gid           = peer.gid;
        r.sgid_index         = ctx_->gid_index();
        r.dest_lid           = peer.lid;
        r.is_global          = ctx_->is_roce();
        r.port               = ctx_->port();
        r.service_level      = env.service_level;
        r.max_rd_atomic      = env.max_rd_atomic;
        r.max_dest_rd_atomic = env.max_dest_rd_atomic;
        if (ctx_->dev().qp_to_rtr(ch.lanes[i].qp, r) != 0) {
            SLIME_LOG_ERROR("queue pair ", ch.lanes[i].qpn, " failed to reach RTR");
            return -1;
        }
        if (ctx_->dev().qp_to_rts(ch.lanes[i].qp, r) != 0) {
            SLIME_LOG_ERROR("queue pair ", ch.lanes[i].qpn, " failed to reach RTS");
            return -1;
        }
    }
    return 0;
}

void RdmaEndpoint::post_window(Channel& ch, int channel_id)
{
    std::vector<RecvWr> wrs(ch.recv_window);
    for (size_t lane = 0; lane < ch.lanes.size(); ++lane) {
        for (int i = 0; i < ch.recv_window; ++i) {
            RecvWr& w = wrs[i];
            w         = RecvWr{};
            if (channel_id == CH_META) {
                w.wr_id      = make_wr_id(K_META_RECV, 0, static_cast<uint32_t>(i));
                w.sge.addr   = meta_mr_.addr + static_cast<uint64_t>(i) * sizeof(MetaMsg);
                w.sge.length = sizeof(MetaMsg);
                w.sge.lkey   = static_cast<uint32_t>(meta_mr_.lkey);
            }
            else {
                w.wr_id = make_wr_id(K_WINDOW_RECV, 0, (static_cast<uint32_t>(channel_id) << 16) | static_cast<uint32_t>(lane));
            }
        }
        int posted = 0;
        if (ctx_->dev().post_recv(ch.lanes[lane].qp, wrs.data(), ch.recv_window, &posted) != 0)
            SLIME_LOG_WARN("only ", posted, " of ", ch.recv_window, " receives could be posted on queue pair ", ch.lanes[lane].qpn);
    }
}

int RdmaEndpoint::connect(const Json& remote)
{
    if (connected_.load()) return 0;
    if (remote["kind"].string_or("rdma") != "rdma") {
        SLIME_LOG_ERROR("peer endpoint is of kind ", remote["kind"].string_or("?"), ", not rdma");
        return -1;
    }
    // receives go in before the queue pairs can receive, so the peer's first message never finds an empty queue
    post_window(ch_[CH_IO], CH_IO);
    post_window(ch_[CH_MSG], CH_MSG);
    post_window(ch_[CH_META], CH_META);
    if (connect_channel(ch_[CH_IO], remote["io"], "io") != 0 || connect_channel(ch_[CH_MSG], remote["msg"], "msg") != 0
        || connect_channel(ch_[CH_META], remote["meta"], "meta") != 0)
        return -1;
    if (remote.contains("mr_info") && remote["mr_info"].is_object())
        for (auto& kv : remote["mr_info"].fields()) register_remote_memory_region(kv.first, kv.second);
    connected_.store(true);
    return 0;
}

bool RdmaEndpoint::ensure_local(uintptr_t addr, uint64_t bytes, MemoryRegion& out)
{
    int32_t h = local_pool_->get_mr_handle(addr);
    if (h >= 0 && local_pool_->get_mr(h, out) && out.length >= bytes) return true;
    h = local_pool_->register_memory_region(addr, bytes, std::nullopt);
    return h >= 0 && local_pool_->get_mr(h, out);
}

void RdmaEndpoint::wake_worker()
{
    if (worker_) worker_->wake();
}

// ---------------------------------------------------------------------------------------------------
// building work requests

void RdmaEndpoint::build_striped(TxOp& op, WrOp data_op, uint64_t local_addr, uint32_t lkey, uint64_t remote_addr, uint32_t rkey,
                                 uint64_t length, size_t& rr)
{
    const uint64_t max_len = std::max<uint64_t>(1, std::min<uint64_t>(engine_env().max_length_per_assignment, 1ull << 30));
    for (uint64_t done = 0; done < length;) {
        const uint64_t chunk = std::min(max_len, length - done);
        if (chunk >= stripe_min_bytes_ && num_qp_ > 1) {
            const uint64_t per = (chunk + num_qp_ - 1) / num_qp_;
            for (int lane = 0; lane < num_qp_; ++lane) {
                const uint64_t lo = static_cast<uint64_t>(lane) * per;
                if (lo >= chunk) break;
                const uint64_t n = std::min(per, chunk - lo);
                SendWr w;
                w.op          = data_op;
                w.sge         = Sge{local_addr + done + lo, static_cast<uint32_t>(n), lkey};
                w.remote_addr = remote_addr + done + lo;
                w.rkey        = rkey;
                op.lane_wrs[lane].push_back(w);
            }
        }
        else {
            SendWr w;
            w.op          = data_op;
            w.sge         = Sge{local_addr + done, static_cast<uint32_t>(chunk), lkey};
            w.remote_addr = remote_addr + done;
            w.rkey        = rkey;
            op.lane_wrs[rr++ % num_qp_].push_back(w);
        }
        done += chunk;
    }
}

// Signal marks, immediates and work-request ids; called once all data work requests are in place.
void RdmaEndpoint::finish_lanes(TxOp& op, bool with_imm, uint32_t imm)
{
    for (int lane = 0; lane < num_qp_; ++lane) {
        auto& wrs = op.lane_wrs[lane];
        if (with_imm) {
            if (wrs.empty() || wrs.back().op != WrOp::WRITE) {
                SendWr w;
                w.op = WrOp::WRITE_WITH_IMM;
                wrs.push_back(w);
            }
            wrs.back().op  = WrOp::WRITE_WITH_IMM;
            wrs.back().imm = imm;
        }
        for (size_t i = 0; i < wrs.size(); ++i) wrs[i].signaled = ((i + 1) % kSignalEvery == 0) || i + 1 == wrs.size();
    }
}

std::shared_ptr<ReadWriteFuture> RdmaEndpoint::submit_one_sided(OpCode opcode, const std::vector<assign_tuple_t>& assign, int32_t imm,
                                                                void* stream)
{
    const uint32_t mask = num_qp_ >= 32 ? 0xffffffffu : ((1u << num_qp_) - 1);
    auto           st   = make_op_state(mask, opcode);
    st->link_id         = ctx_->obs_link();
    if (engine_env().with_time_trace) st->trace_start_ns.store(monotonic_ns());
    auto fut = std::make_shared<ReadWriteFuture>(st);
    auto fail_now = [&](int32_t status) {
        st->fail(status);
        obs::record_submit(st->link_id, obs::op_index(opcode), assign.size(), 0);
        complete_state(st);
        st->signal->force_complete();
        return fut;
    };
    if (shut_.load() || !connected_.load()) return fail_now(FAILED);

    TxOp op;
    op.state   = st;
    op.channel = CH_IO;
    op.lane_wrs.resize(num_qp_);
    op.cursor.assign(num_qp_, 0);
    op.slot.assign(num_qp_, -1);
    const WrOp data_op = opcode == OpCode::READ ? WrOp::READ : WrOp::WRITE;
    uint64_t   bytes   = 0;
    {
        std::lock_guard<std::mutex> g(fifo_mu_);
        for (const auto& t : assign) {
            const Assignment a(t);
            MemoryRegion     lm, rm;
            if (!local_pool_->get_mr(static_cast<int32_t>(a.mr_key), lm) || !lm.contains(a.source_offset, a.length)
                || !remote_pool_->get_remote_mr(static_cast<int32_t>(a.remote_mr_key), rm) || !rm.contains(a.target_offset, a.length)) {
                SLIME_LOG_ERROR("assignment outside its registered regions: ", a.dump());
                return fail_now(FAILED);
            }
            build_striped(op, data_op, lm.addr + a.source_offset, static_cast<uint32_t>(lm.lkey), rm.addr + a.target_offset,
                          static_cast<uint32_t>(rm.rkey), a.length, rr_lane_);
            bytes += a.length;
        }
        finish_lanes(op, opcode == OpCode::WRITE_WITH_IMM, static_cast<uint32_t>(imm));
        st->bytes = bytes;
        obs::record_submit(st->link_id, obs::op_index(opcode), assign.size(), bytes);
        if (stream != nullptr && !engine_env().bypass_device_signal) st->signal->bind_stream(stream);
        st->signal->record_gpu_ready();
        track(st);
        tx_fifo_[CH_IO].push_back(std::move(op));
    }
    wake_worker();
    return fut;
}

std::shared_ptr<ReadWriteFuture> RdmaEndpoint::read(const std::vector<assign_tuple_t>& assign, void* stream)
{
    return submit_one_sided(OpCode::READ, assign, 0, stream);
}

std::shared_ptr<ReadWriteFuture> RdmaEndpoint::write(const std::vector<assign_tuple_t>& assign, void* stream)
{
    return submit_one_sided(OpCode::WRITE, assign, 0, stream);
}

std::shared_ptr<ReadWriteFuture> RdmaEndpoint::write_with_imm(const std::vector<assign_tuple_t>& assign, int32_t imm_data, void* stream)
{
    return submit_one_sided(OpCode::WRITE_WITH_IMM, assign, imm_data, stream);
}

std::shared_ptr<ImmRecvFuture> RdmaEndpoint::imm_recv(void*)
{
    auto st     = make_op_state(1, OpCode::RECV);
    st->link_id = ctx_->obs_link();
    if (engine_env().with_time_trace) st->trace_start_ns.store(monotonic_ns());
    auto fut = std::make_shared<ImmRecvFuture>(st);
    obs::record_submit(st->link_id, obs::OP_IMM_RECV, 1, 0);
    std::lock_guard<std::mutex> g(imm_mu_);
    if (shut_.load()) {
        st->fail(FAILED);
        st->signal->force_complete();
    }
    else if (!imm_events_.empty()) {
        st->imm_data.store(static_cast<int32_t>(imm_events_.front()));
        imm_events_.pop_front();
        st->trace_end_ns.store(monotonic_ns());
        obs::record_complete(st->link_id, obs::OP_IMM_RECV, 0);
        st->signal->set_comm_done(0);
    }
    else {
        imm_waiters_.push_back(st);
    }
    return fut;
}

std::shared_ptr<SendFuture> RdmaEndpoint::send(const chunk_tuple_t& chunk, void* stream)
{
    const uint32_t mask = num_qp_ >= 32 ? 0xffffffffu : ((1u << num_qp_) - 1);
    auto           st   = make_op_state(mask, OpCode::SEND);
    st->link_id         = ctx_->obs_link();
    st->bytes           = std::get<2>(chunk);
    auto fut            = std::make_shared<SendFuture>(st);
    obs::record_submit(st->link_id, obs::OP_SEND, 1, st->bytes);
    MemoryRegion mr;
    const uintptr_t base = std::get<0>(chunk);
    if (shut_.load() || !connected_.load() || !ensure_local(base, std::get<1>(chunk) + std::get<2>(chunk), mr)) {
        st->fail(FAILED);
        complete_state(st);
        st->signal->force_complete();
        return fut;
    }
    SendOp op;
    op.state  = st;
    op.addr   = base + std::get<1>(chunk);
    op.length = std::get<2>(chunk);
    op.lkey   = static_cast<uint32_t>(mr.lkey);
    if (stream != nullptr && !engine_env().bypass_device_signal) st->signal->bind_stream(stream);
    st->signal->record_gpu_ready();
    track(st);
    {
        std::lock_guard<std::mutex> g(fifo_mu_);
        send_fifo_.push_back(std::move(op));
    }
    wake_worker();
    return fut;
}

std::shared_ptr<RecvFuture> RdmaEndpoint::recv(const chunk_tuple_t& chunk, void* stream)
{
    auto st     = make_op_state(1, OpCode::RECV);
    st->link_id = ctx_->obs_link();
    st->bytes   = std::get<2>(chunk);
    auto fut    = std::make_shared<RecvFuture>(st);
    obs::record_submit(st->link_id, obs::OP_RECV, 1, st->bytes);
    MemoryRegion mr;
    const uintptr_t base = std::get<0>(chunk);
    if (shut_.load() || !connected_.load() || !ensure_local(base, std::get<1>(chunk) + std::get<2>(chunk), mr)) {
        st->fail(FAILED);
        complete_state(st);
        st->signal->force_complete();
        return fut;
    }
    RecvOp op;
    op.state  = st;
    op.addr   = base + std::get<1>(chunk);
    op.length = std::get<2>(chunk);
    op.rkey   = static_cast<uint32_t>(mr.rkey);
    if (stream != nullptr && !engine_env().bypass_device_signal) st->signal->bind_stream(stream);
    st->signal->record_gpu_ready();
    track(st);
    {
        std::lock_guard<std::mutex> g(fifo_mu_);
        op.seq = recv_seq_++;
        recv_fifo_.push_back(std::move(op));
    }
    wake_worker();
    return fut;
}

// ---------------------------------------------------------------------------------------------------
// progress thread

void RdmaEndpoint::track(const std::shared_ptr<EndpointOpState>& st)
{
    std::lock_guard<std::mutex> g(inflight_mu_);
    inflight_[st.get()] = st;
}

void RdmaEndpoint::complete_state(const std::shared_ptr<EndpointOpState>& st)
{
    if (st->obs_completed.exchange(true)) return;
    {
        std::lock_guard<std::mutex> g(inflight_mu_);
        inflight_.erase(st.get());
    }
    st->trace_end_ns.store(monotonic_ns());
    obs::OpIndex oi = obs::op_index(st->opcode);
    if (st->completion_status.load() == SUCCESS)
        obs::record_complete(st->link_id, oi, st->bytes);
    else
        obs::record_fail(st->link_id, oi, st->bytes);
}

void RdmaEndpoint::lane_done(TxLane& tl, uint32_t slot)
{
    std::shared_ptr<EndpointOpState> st = std::move(tl.state);
    const int lane = tl.lane;
    tl.state.reset();
    free_slots_.try_push(slot);
    if (!st) return;
    // the accounting latch goes first so that a waiter that wakes up sees final counters
    const uint32_t after = st->signal->get_comm_done_mask() | (1u << lane);
    if ((after & st->expected_mask) == st->expected_mask) complete_state(st);
    st->signal->set_comm_done(lane);
}

void RdmaEndpoint::fail_tx(TxOp& op)
{
    op.state->fail(FAILED);
    complete_state(op.state);
    op.state->signal->force_complete();
}

int RdmaEndpoint::post_tx(int c)
{
    if (!cur_tx_[c]) {
        std::lock_guard<std::mutex> g(fifo_mu_);
        if (tx_fifo_[c].empty()) return 0;
        cur_tx_[c] = std::move(tx_fifo_[c].front());
        tx_fifo_[c].pop_front();
    }
    TxOp& op = *cur_tx_[c];
    if (!op.state->signal->is_gpu_ready()) return 0;
    Channel& ch = ch_[c];
    if (!op.leased) {
        int need = 0;
        for (auto& w : op.lane_wrs) need += w.empty() ? 0 : 1;
        std::vector<uint32_t> got;
        uint32_t              s = 0;
        while (static_cast<int>(got.size()) < need && free_slots_.try_pop(s)) got.push_back(s);
        if (static_cast<int>(got.size()) < need) {
            for (uint32_t x : got) free_slots_.try_push(x);
            return 0;
        }
        size_t gi = 0;
        bool   any = false;
        for (int lane = 0; lane < num_qp_; ++lane) {
            auto& wrs = op.lane_wrs[lane];
            if (wrs.empty()) continue;
            any             = true;
            const uint32_t slot = got[gi++];
            TxLane&        tl   = tx_slots_[slot];
            tl.state   = op.state;
            tl.lane    = lane;
            tl.channel = c;
            int signaled = 0, since = 0;
            for (auto& w : wrs) {
                ++since;
                if (w.signaled) {
                    w.wr_id = make_wr_id(K_TX, static_cast<uint32_t>(since), slot);
                    since   = 0;
                    ++signaled;
                }
                else {
                    w.wr_id = make_wr_id(K_TX_UNSIGNALED, 0, slot);
                }
            }
            tl.outstanding.store(signaled, std::memory_order_release);
            op.slot[lane] = static_cast<int32_t>(slot);
            signaled_wrs_.fetch_add(signaled, std::memory_order_relaxed);
        }
        op.leased = true;
        // lanes without work are done from the start
        for (int lane = 0; lane < num_qp_; ++lane) {
            if (!op.lane_wrs[lane].empty()) continue;
            const uint32_t after = op.state->signal->get_comm_done_mask() | (1u << lane);
            if (!any && (after & op.state->expected_mask) == op.state->expected_mask) complete_state(op.state);
            op.state->signal->set_comm_done(lane);
        }
    }
    int  work     = 0;
    bool all_done = true;
    const obs::OpIndex oi = obs::op_index(op.state->opcode);
    for (int lane = 0; lane < num_qp_; ++lane) {
        auto&        wrs       = op.lane_wrs[lane];
        const size_t remaining = wrs.size() - op.cursor[lane];
        if (remaining == 0) continue;
        Lane&     l       = ch.lanes[lane];
        const int credits = l.credits.load(std::memory_order_acquire);
        if (credits <= 0) {
            credit_stalls_.fetch_add(1, std::memory_order_relaxed);
            all_done = false;
            continue;
        }
        const int n = static_cast<int>(std::min<size_t>(remaining, static_cast<size_t>(credits)));
        l.credits.fetch_sub(n, std::memory_order_acq_rel);
        int       posted = 0;
        const int rc     = ctx_->dev().post_send(l.qp, wrs.data() + op.cursor[lane], n, &posted);
        uint64_t  bytes  = 0;
        for (int i = 0; i < posted; ++i) bytes += wrs[op.cursor[lane] + i].sge.length;
        obs::record_post_batch(op.state->link_id, oi, posted, bytes);
        posted_wrs_.fetch_add(posted, std::memory_order_relaxed);
        op.cursor[lane] += posted;
        work += posted;
        if (rc != 0) {
            // nothing after the failing work request will ever complete: settle the lane here
            obs::record_post_failure(op.state->link_id, oi);
            l.credits.fetch_add(n - posted, std::memory_order_acq_rel);
            op.state->fail(FAILED);
            int unposted_signaled = 0;
            for (size_t i = op.cursor[lane]; i < wrs.size(); ++i) unposted_signaled += wrs[i].signaled ? 1 : 0;
            op.cursor[lane]     = wrs.size();
            const uint32_t slot = static_cast<uint32_t>(op.slot[lane]);
            TxLane&        tl   = tx_slots_[slot];
            if (unposted_signaled > 0 && tl.outstanding.fetch_sub(unposted_signaled, std::memory_order_acq_rel) == unposted_signaled)
                lane_done(tl, slot);
            work += 1;
        }
        if (op.cursor[lane] < wrs.size()) all_done = false;
    }
    if (all_done) cur_tx_[c].reset();
    return work;
}

// Announce receive buffers that are ready: one inline meta message per recv.
int RdmaEndpoint::progress_recv()
{
    int work = 0;
    for (;;) {
        RecvOp op;
        {
            std::lock_guard<std::mutex> g(fifo_mu_);
            if (recv_fifo_.empty() || !recv_fifo_.front().state->signal->is_gpu_ready()) return work;
            Lane& ml = ch_[CH_META].lanes[0];
            if (ml.credits.load(std::memory_order_acquire) <= 0) return work;
            ml.credits.fetch_sub(1, std::memory_order_acq_rel);
            op = std::move(recv_fifo_.front());
            recv_fifo_.pop_front();
        }
        MetaMsg m;
        memset(&m, 0, sizeof(m));
        m.seq    = op.seq;
        m.addr   = op.addr;
        m.length = op.length;
        m.rkey   = op.rkey;
        {
            std::lock_guard<std::mutex> g(imm_mu_);
            announced_.push_back(op);  // before the message leaves: the answer may come at once
        }
        SendWr w;
        w.op          = WrOp::SEND;
        w.inline_data = true;
        w.signaled    = true;
        w.wr_id       = make_wr_id(K_META_SEND, 1, 0);
        w.sge         = Sge{reinterpret_cast<uint64_t>(&m), sizeof(MetaMsg), 0};
        int posted    = 0;
        if (ctx_->dev().post_send(ch_[CH_META].lanes[0].qp, &w, 1, &posted) != 0) {
            ch_[CH_META].lanes[0].credits.fetch_add(1, std::memory_order_acq_rel);
            {
                std::lock_guard<std::mutex> g(imm_mu_);
                for (auto it = announced_.begin(); it != announced_.end(); ++it)
                    if (it->state == op.state) {
                        announced_.erase(it);
                        break;
                    }
            }
            op.state->fail(FAILED);
            complete_state(op.state);
            op.state->signal->force_complete();
        }
        ++work;
    }
}

// Pair the oldest send with the oldest announcement and queue its payload on the msg channel.
int RdmaEndpoint::progress_send()
{
    int work = 0;
    for (;;) {
        std::lock_guard<std::mutex> g(fifo_mu_);
        if (send_fifo_.empty() || !send_fifo_.front().state->signal->is_gpu_ready()) return work;
        MetaMsg m;
        {
            std::lock_guard<std::mutex> gi(imm_mu_);
            if (metas_.empty()) return work;
            m = metas_.front();
            metas_.pop_front();
        }
        SendOp op = std::move(send_fifo_.front());
        send_fifo_.pop_front();
        const bool     overflow = op.length > m.length;
        const uint64_t n        = std::min<uint64_t>(op.length, m.length);
        TxOp tx;
        tx.state   = op.state;
        tx.channel = CH_MSG;
        tx.lane_wrs.resize(num_qp_);
        tx.cursor.assign(num_qp_, 0);
        tx.slot.assign(num_qp_, -1);
        build_striped(tx, WrOp::WRITE, op.addr, op.lkey, m.addr, m.rkey, n, rr_lane_);
        finish_lanes(tx, true, (static_cast<uint32_t>(m.seq) & ~kOverflowBit) | (overflow ? kOverflowBit : 0));
        if (overflow) op.state->fail(ASSIGNMENT_BATCH_OVERFLOW);
        tx_fifo_[CH_MSG].push_back(std::move(tx));
        ++work;
    }
}

int RdmaEndpoint::process()
{
    if (shut_.load(std::memory_order_acquire) || !connected_.load(std::memory_order_acquire)) return 0;
    std::unique_lock<std::mutex> g(proc_mu_, std::try_to_lock);
    if (!g.owns_lock()) return 0;
    int work = 0;
    work += post_tx(CH_IO);
    work += progress_recv();
    work += progress_send();
    work += post_tx(CH_MSG);
    return work;
}

// ---------------------------------------------------------------------------------------------------
// completion thread

void RdmaEndpoint::repost_window(int channel_id, int lane)
{
    RecvWr w;
    w.wr_id = make_wr_id(K_WINDOW_RECV, 0, (static_cast<uint32_t>(channel_id) << 16) | static_cast<uint32_t>(lane));
    ctx_->dev().post_recv(ch_[channel_id].lanes[lane].qp, &w, 1, nullptr);
}

// The k-th immediate has arrived on every lane of the channel (imm_mu_ held).
void RdmaEndpoint::deliver_group(int channel_id, uint32_t imm)
{
    if (channel_id == CH_IO) {
        if (imm_waiters_.empty()) {
            imm_events_.push_back(imm);
            return;
        }
        auto st = std::move(imm_waiters_.front());
        imm_waiters_.pop_front();
        st->imm_data.store(static_cast<int32_t>(imm));
        st->trace_end_ns.store(monotonic_ns());
        obs::record_complete(st->link_id, obs::OP_IMM_RECV, 0);
        st->signal->set_comm_done(0);
        return;
    }
    if (announced_.empty()) {
        SLIME_LOG_WARN("payload arrived without a matching recv (sends and recvs out of order?)");
        return;
    }
    RecvOp op = std::move(announced_.front());
    announced_.pop_front();
    if (imm & kOverflowBit) op.state->fail(ASSIGNMENT_BATCH_OVERFLOW);
    complete_state(op.state);
    op.state->signal->set_comm_done(0);
}

void RdmaEndpoint::on_completion(const Completion& wc)
{
    const WrKind   kind   = static_cast<WrKind>(wc.wr_id >> 60);
    const uint32_t refund = static_cast<uint32_t>((wc.wr_id >> 40) & 0xffff);
    const uint32_t index  = static_cast<uint32_t>(wc.wr_id & 0xffffffffu);
    switch (kind) {
        case K_TX: {
            if (index >= kTxSlots) return;
            TxLane& tl = tx_slots_[index];
            ch_[tl.channel].lanes[tl.lane].credits.fetch_add(static_cast<int>(refund), std::memory_order_acq_rel);
            if (wc.status != WC_SUCCESS && tl.state) tl.state->fail(FAILED);
            if (tl.outstanding.fetch_sub(1, std::memory_order_acq_rel) == 1) lane_done(tl, index);
            wake_worker();
            break;
        }
        case K_TX_UNSIGNALED: {  // only failures produce these
            if (index < kTxSlots && wc.status != WC_SUCCESS) {
                auto st = tx_slots_[index].state;
                if (st) st->fail(FAILED);
            }
            break;
        }
        case K_WINDOW_RECV: {
            if (wc.status != WC_SUCCESS) return;  // flushed at shutdown
            const int channel_id = static_cast<int>(index >> 16), lane = static_cast<int>(index & 0xffff);
            if (channel_id > CH_MSG || lane >= static_cast<int>(ch_[channel_id].lanes.size())) return;
            if (wc.has_imm) {
                std::lock_guard<std::mutex> g(imm_mu_);
                Channel& ch = ch_[channel_id];
                ch.lanes[lane].imms.push_back(wc.imm);
                bool all = true;
                for (auto& l : ch.lanes) all = all && !l.imms.empty();
                if (all) {
                    uint32_t imm = wc.imm;
                    for (auto& l : ch.lanes) {
                        imm = l.imms.front();
                        l.imms.pop_front();
                    }
                    deliver_group(channel_id, imm);
                }
            }
            if (!shut_.load(std::memory_order_acquire)) repost_window(channel_id, lane);
            break;
        }
        case K_META_SEND: {
            ch_[CH_META].lanes[0].credits.fetch_add(static_cast<int>(refund), std::memory_order_acq_rel);
            if (wc.status != WC_SUCCESS && wc.status != WC_WR_FLUSH_ERR) SLIME_LOG_ERROR("meta message failed with status ", wc.status);
            wake_worker();
            break;
        }
        case K_META_RECV: {
            if (wc.status != WC_SUCCESS || static_cast<int>(index) >= meta_depth_) return;
            MetaMsg m;
            memcpy(&m, meta_buf_.data() + static_cast<size_t>(index) * sizeof(MetaMsg), sizeof(m));
            {
                std::lock_guard<std::mutex> g(imm_mu_);
                metas_.push_back(m);
            }
            if (!shut_.load(std::memory_order_acquire)) {
                RecvWr w;
                w.wr_id      = make_wr_id(K_META_RECV, 0, index);
                w.sge.addr   = meta_mr_.addr + static_cast<uint64_t>(index) * sizeof(MetaMsg);
                w.sge.length = sizeof(MetaMsg);
                w.sge.lkey   = static_cast<uint32_t>(meta_mr_.lkey);
                ctx_->dev().post_recv(ch_[CH_META].lanes[0].qp, &w, 1, nullptr);
            }
            wake_worker();
            break;
        }
        default: break;
    }
}

// ---------------------------------------------------------------------------------------------------
// teardown

void RdmaEndpoint::cancel_all()
{
    std::lock_guard<std::mutex> gp(proc_mu_);
    std::vector<std::shared_ptr<EndpointOpState>> victims;
    {
        std::lock_guard<std::mutex> g(fifo_mu_);
        for (auto& q : tx_fifo_) {
            for (auto& op : q) victims.push_back(op.state);
            q.clear();
        }
        for (auto& op : recv_fifo_) victims.push_back(op.state);
        recv_fifo_.clear();
        for (auto& op : send_fifo_) victims.push_back(op.state);
        send_fifo_.clear();
    }
    for (auto& cur : cur_tx_) {
        if (cur) victims.push_back(cur->state);
        // lanes already leased stay with their slots: late completions release them
        cur.reset();
    }
    {
        std::lock_guard<std::mutex> g(imm_mu_);
        for (auto& st : imm_waiters_) victims.push_back(st);
        imm_waiters_.clear();
        for (auto& op : announced_) victims.push_back(op.state);
        announced_.clear();
    }
    {
        // operations whose work requests are already with the device: their lane slots are released by the
        // completions (or flushes) that are still to come; here they are only settled towards the caller
        std::lock_guard<std::mutex> g(inflight_mu_);
        for (auto& kv : inflight_)
            if (auto st = kv.second.lock()) victims.push_back(st);
    }
    for (auto& st : victims) {
        const uint32_t done = st->signal->get_comm_done_mask();
        if ((done & st->expected_mask) == st->expected_mask) continue;  // finished in the meantime
        st->fail(FAILED);
        complete_state(st);
        st->signal->force_complete();
    }
}

void RdmaEndpoint::shutdown()
{
    if (shut_.exchange(true)) return;
    if (worker_) worker_->remove(this);
    cancel_all();
    connected_.store(false);
    {
        std::lock_guard<std::mutex> gp(proc_mu_);
        for (auto& ch : ch_)
            for (auto& l : ch.lanes) {
                if (l.qp) ctx_->dev().destroy_qp(l.qp);
                l.qp = 0;
            }
    }
    for (auto& ch : ch_)
        for (auto& l : ch.lanes) ctx_->remove_sink(l.qpn);
    // user regions live in the context-wide pool and outlive this endpoint; its control ring does not
    if (own_pool_) own_pool_->unregister_memory_region(meta_name_);
}

}  // namespace rdma
}  // namespace slime
