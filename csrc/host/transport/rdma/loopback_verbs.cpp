// Software reliable-connected fabric inside one process (the "loopback" verbs provider).
//
// What it models, because the layers above depend on it:
//   * queue pairs with RESET -> INIT -> RTR -> RTS and an error state; per queue pair FIFO execution
//     by one engine thread (so ordering holds inside a queue pair and NOT across queue pairs);
//   * memory keys with bounds checks on both sides; a bad key fails the work request with the verbs
//     status, moves the queue pair to the error state and flushes everything queued behind it;
//   * receive queues: SEND and WRITE_WITH_IMM consume a posted receive; none posted means
//     receiver-not-ready and the work request is retried (counted in loopback_rnr_events);
//   * completion queues with polling and arm-then-sleep events; unsignaled work requests complete
//     silently unless they fail;
//   * inline sends copy the payload at post time.
// What it does not model: packets, PSNs, MTU, timeouts, atomics, shared receive queues.
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>
#include <unordered_map>

#include "transport/rdma/verbs.h"

namespace slime {
namespace rdma {
namespace {

struct LoMr {
    uintptr_t addr = 0;
    uint64_t  len  = 0;
    uint32_t  key  = 0;
};

struct LoCq {
    std::mutex              mu;
    std::condition_variable cv;
    std::deque<Completion>  q;
    uint64_t                pushed = 0;

    void push(const Completion& c)
    {
        {
            std::lock_guard<std::mutex> g(mu);
            q.push_back(c);
            ++pushed;
        }
        cv.notify_all();
    }
};

struct QueuedSend {
    SendWr               wr;
    std::vector<uint8_t> inline_payload;
};

struct LoQp {
    enum State { RESET, INIT, RTR, RTS, ERR };
    uint32_t               qpn = 0;
    std::shared_ptr<LoCq>  cq;
    QpCaps                 caps;
    State                  state    = RESET;
    uint32_t               dest_qpn = 0;
    std::deque<QueuedSend> sq;
    std::deque<RecvWr>     rq;
};

struct InjectedError {
    WrOp op;
    int  status;
    int  count;
};

class Fabric {
public:
    static Fabric& get()
    {
        static Fabric* f = new Fabric();  // lives until process exit; the engine thread is detached
        return *f;
    }

    std::mutex                                          mu;  // guards every map and every queue of every queue pair
    std::condition_variable                             cv;
    std::unordered_map<uint32_t, std::shared_ptr<LoQp>> qps;
    std::unordered_map<uint32_t, LoMr>                  mrs;
    std::unordered_map<uint64_t, std::shared_ptr<LoCq>> cqs;
    std::vector<InjectedError>                          injected;
    uint32_t                                            next_qpn = 0x100;
    uint32_t                                            next_key = 0x1000;
    uint64_t                                            next_pd  = 1;
    uint64_t                                            pending  = 0;  // queued send work requests over all queue pairs
    std::atomic<uint64_t>                               executed{0}, rnr{0};

    bool key_covers(uint32_t key, uint64_t addr, uint64_t len) const
    {
        auto it = mrs.find(key);
        if (it == mrs.end()) return false;
        return addr >= it->second.addr && len <= it->second.len && addr - it->second.addr <= it->second.len - len;
    }

    // Moves a queue pair to the error state and flushes its queues (caller holds mu).
    void fail_qp(LoQp& qp)
    {
        qp.state = LoQp::ERR;
        for (auto& s : qp.sq) {
            Completion c;
            c.wr_id  = s.wr.wr_id;
            c.status = WC_WR_FLUSH_ERR;
            c.qp_num = qp.qpn;
            qp.cq->push(c);
        }
        pending -= qp.sq.size();
        qp.sq.clear();
        for (auto& r : qp.rq) {
            Completion c;
            c.wr_id  = r.wr_id;
            c.status = WC_WR_FLUSH_ERR;
            c.op     = WcOp::RECV;
            c.qp_num = qp.qpn;
            qp.cq->push(c);
        }
        qp.rq.clear();
    }

private:
    Fabric() { std::thread([this] { run(); }).detach(); }

    int injected_status(WrOp op)
    {
        for (auto& e : injected)
            if (e.op == op && e.count > 0) {
                --e.count;
                return e.status;
            }
        return WC_SUCCESS;
    }

    // Executes the head work request of one queue pair. Returns false when it must be retried later
    // (receiver not ready). Caller holds mu; the copy itself runs under the lock too, which keeps a
    // destination region from being deregistered in mid-copy.
    bool execute_head(LoQp& qp)
    {
        QueuedSend& qs = qp.sq.front();
        SendWr&     wr = qs.wr;
        int         status = injected_status(wr.op);
        const void* src    = wr.inline_data ? qs.inline_payload.data() : reinterpret_cast<const void*>(wr.sge.addr);
        LoQp*       dst    = nullptr;
        if (auto it = qps.find(qp.dest_qpn); it != qps.end() && it->second->state >= LoQp::RTR && it->second->state != LoQp::ERR)
            dst = it->second.get();
        if (status == WC_SUCCESS && dst == nullptr) status = WC_RETRY_EXC_ERR;
        if (status == WC_SUCCESS && wr.sge.length > 0 && !wr.inline_data && !key_covers(wr.sge.lkey, wr.sge.addr, wr.sge.length))
            status = WC_LOC_PROT_ERR;
        const bool one_sided = wr.op == WrOp::WRITE || wr.op == WrOp::WRITE_WITH_IMM || wr.op == WrOp::READ;
        if (status == WC_SUCCESS && one_sided && wr.sge.length > 0 && !key_covers(wr.rkey, wr.remote_addr, wr.sge.length))
            status = WC_REM_ACCESS_ERR;
        const bool needs_recv = wr.op == WrOp::SEND || wr.op == WrOp::SEND_WITH_IMM || wr.op == WrOp::WRITE_WITH_IMM;
        if (status == WC_SUCCESS && needs_recv && dst->rq.empty()) {
            rnr.fetch_add(1, std::memory_order_relaxed);
            return false;
        }
        Completion recv_c;
        bool       have_recv_c = false;
        if (status == WC_SUCCESS) {
            switch (wr.op) {
                case WrOp::WRITE:
                case WrOp::WRITE_WITH_IMM:
                    if (wr.sge.length) memcpy(reinterpret_cast<void*>(wr.remote_addr), src, wr.sge.length);
                    break;
                case WrOp::READ:
                    if (wr.sge.length) memcpy(reinterpret_cast<void*>(wr.sge.addr), reinterpret_cast<const void*>(wr.remote_addr), wr.sge.length);
                    break;
                case WrOp::SEND:
                case WrOp::SEND_WITH_IMM: {
                    const RecvWr& r = dst->rq.front();
                    if (wr.sge.length > r.sge.length || (wr.sge.length > 0 && !key_covers(r.sge.lkey, r.sge.addr, wr.sge.length)))
                        status = WC_REM_ACCESS_ERR;  // receive buffer too small / not registered
                    else if (wr.sge.length)
                        memcpy(reinterpret_cast<void*>(r.sge.addr), src, wr.sge.length);
                    break;
                }
            }
            if (status == WC_SUCCESS && needs_recv) {
                recv_c.wr_id    = dst->rq.front().wr_id;
                recv_c.op       = wr.op == WrOp::WRITE_WITH_IMM ? WcOp::RECV_WITH_IMM : WcOp::RECV;
                recv_c.has_imm  = wr.op != WrOp::SEND;
                recv_c.imm      = wr.imm;
                recv_c.byte_len = wr.sge.length;
                recv_c.qp_num   = dst->qpn;
                have_recv_c     = true;
                dst->rq.pop_front();
            }
        }
        executed.fetch_add(1, std::memory_order_relaxed);
        if (status != WC_SUCCESS) {
            Completion c;
            c.wr_id  = wr.wr_id;
            c.status = status;
            c.qp_num = qp.qpn;
            qp.cq->push(c);
            qp.sq.pop_front();
            --pending;
            fail_qp(qp);
            return true;
        }
        if (wr.signaled) {
            Completion c;
            c.wr_id    = wr.wr_id;
            c.op       = wr.op == WrOp::READ ? WcOp::READ : (one_sided ? WcOp::WRITE : WcOp::SEND);
            c.byte_len = wr.sge.length;
            c.qp_num   = qp.qpn;
            qp.cq->push(c);
        }
        qp.sq.pop_front();
        --pending;
        if (have_recv_c) dst->cq->push(recv_c);
        return true;
    }

    void run()
    {
        std::unique_lock<std::mutex> g(mu);
        for (;;) {
            cv.wait(g, [&] { return pending > 0; });
            bool progressed = false;
            // snapshot of the queue pairs with work; each gets a burst so one long batch cannot starve the rest
            std::vector<std::shared_ptr<LoQp>> work;
            for (auto& kv : qps)
                if (!kv.second->sq.empty() && kv.second->state == LoQp::RTS) work.push_back(kv.second);
            for (auto& qp : work) {
                for (int burst = 0; burst < 64 && !qp->sq.empty() && qp->state == LoQp::RTS; ++burst) {
                    if (!execute_head(*qp)) break;
                    progressed = true;
                }
            }
            if (!progressed) {
                // only receiver-not-ready heads (or queue pairs not yet connected): back off briefly
                g.unlock();
                std::this_thread::sleep_for(std::chrono::microseconds(50));
                g.lock();
            }
        }
    }
};

class LoDevice final: public VerbsDevice {
public:
    LoDevice(std::string name, LinkLayer ll): name_(std::move(name)), link_(ll) {}

    std::string name() const override { return name_; }
    DeviceAttr  query_device() override
    {
        DeviceAttr a;
        a.max_cqe        = 1 << 20;
        a.max_qp_wr      = 32768;
        a.max_sge        = 16;
        a.max_qp_rd_atom = 16;
        return a;
    }
    PortAttr query_port(int port) override
    {
        PortAttr p;
        p.active      = port == 1;
        p.lid         = link_ == LinkLayer::IB ? 7 : 0;
        p.active_mtu  = 5;
        p.gid_tbl_len = 4;
        p.link_layer  = link_;
        return p;
    }
    bool query_gid(int, int index, Gid& out) override
    {
        if (index < 0 || index >= 4) return false;
        out.fill(0);
        if (index == 0) {  // link-local style entry
            out[0] = 0xfe;
            out[1] = 0x80;
            out[15] = 1;
        }
        else {  // IPv4-mapped 127.0.0.1
            out[10] = out[11] = 0xff;
            out[12] = 127;
            out[15] = 1;
        }
        return true;
    }
    int find_roce_v2_gid(int, int) override { return link_ == LinkLayer::ETHERNET ? 1 : -1; }

    uint64_t alloc_pd() override
    {
        std::lock_guard<std::mutex> g(F().mu);
        return F().next_pd++;
    }
    void dealloc_pd(uint64_t) override {}
    bool reg_mr(uint64_t, uintptr_t addr, uint64_t len, MrKeys& out) override
    {
        std::lock_guard<std::mutex> g(F().mu);
        const uint32_t key = F().next_key++;
        F().mrs[key]       = LoMr{addr, len, key};
        out.handle = key;
        out.lkey = out.rkey = key;
        return true;
    }
    void dereg_mr(uint64_t handle) override
    {
        std::lock_guard<std::mutex> g(F().mu);
        F().mrs.erase(static_cast<uint32_t>(handle));
    }

    uint64_t create_cq(int) override
    {
        auto cq = std::make_shared<LoCq>();
        std::lock_guard<std::mutex> g(F().mu);
        const uint64_t h = reinterpret_cast<uint64_t>(cq.get());
        F().cqs[h]       = cq;
        return h;
    }
    void destroy_cq(uint64_t cq) override
    {
        std::lock_guard<std::mutex> g(F().mu);
        F().cqs.erase(cq);
    }
    int poll_cq(uint64_t cq, int max_entries, Completion* out) override
    {
        LoCq* c = reinterpret_cast<LoCq*>(cq);
        std::lock_guard<std::mutex> g(c->mu);
        int n = 0;
        while (n < max_entries && !c->q.empty()) {
            out[n++] = c->q.front();
            c->q.pop_front();
        }
        return n;
    }
    bool wait_cq_event(uint64_t cq, int timeout_ms) override
    {
        LoCq* c = reinterpret_cast<LoCq*>(cq);
        std::unique_lock<std::mutex> g(c->mu);
        return c->cv.wait_for(g, std::chrono::milliseconds(timeout_ms), [&] { return !c->q.empty(); });
    }

    uint64_t create_qp(uint64_t, uint64_t cq, const QpCaps& caps, uint32_t& qp_num_out) override
    {
        std::lock_guard<std::mutex> g(F().mu);
        auto it = F().cqs.find(cq);
        if (it == F().cqs.end()) return 0;
        auto qp  = std::make_shared<LoQp>();
        qp->qpn  = F().next_qpn++;
        qp->cq   = it->second;
        qp->caps = caps;
        F().qps[qp->qpn] = qp;
        qp_num_out       = qp->qpn;
        return reinterpret_cast<uint64_t>(qp.get());
    }
    void destroy_qp(uint64_t h) override
    {
        std::lock_guard<std::mutex> g(F().mu);
        LoQp* qp = reinterpret_cast<LoQp*>(h);
        auto  it = F().qps.find(qp->qpn);
        if (it == F().qps.end()) return;
        F().fail_qp(*qp);
        F().qps.erase(it);
    }
    int qp_to_init(uint64_t h, int) override { return set_state(h, LoQp::RESET, LoQp::INIT, 0); }
    int qp_to_rtr(uint64_t h, const QpRoute& r) override { return set_state(h, LoQp::INIT, LoQp::RTR, r.dest_qpn); }
    int qp_to_rts(uint64_t h, const QpRoute&) override
    {
        const int rc = set_state(h, LoQp::RTR, LoQp::RTS, 0);
        F().cv.notify_all();
        return rc;
    }

    int post_send(uint64_t h, const SendWr* wrs, int n, int* n_posted) override
    {
        LoQp* qp = reinterpret_cast<LoQp*>(h);
        int   posted = 0, rc = 0;
        {
            std::lock_guard<std::mutex> g(F().mu);
            if (qp->state != LoQp::RTS) rc = 22;  // EINVAL, like posting to a queue pair that cannot send
            for (; rc == 0 && posted < n; ++posted) {
                if (static_cast<int>(qp->sq.size()) >= qp->caps.max_send_wr) {
                    rc = 12;  // ENOMEM: send queue full
                    break;
                }
                QueuedSend qs;
                qs.wr = wrs[posted];
                if (qs.wr.inline_data) {
                    if (static_cast<int>(qs.wr.sge.length) > qp->caps.max_inline) {
                        rc = 22;
                        break;
                    }
                    const uint8_t* p = reinterpret_cast<const uint8_t*>(qs.wr.sge.addr);
                    qs.inline_payload.assign(p, p + qs.wr.sge.length);
                }
                qp->sq.push_back(std::move(qs));
                ++F().pending;
            }
        }
        if (n_posted) *n_posted = posted;
        if (posted) F().cv.notify_all();
        return rc;
    }
    int post_recv(uint64_t h, const RecvWr* wrs, int n, int* n_posted) override
    {
        LoQp* qp = reinterpret_cast<LoQp*>(h);
        int   posted = 0, rc = 0;
        {
            std::lock_guard<std::mutex> g(F().mu);
            if (qp->state == LoQp::RESET || qp->state == LoQp::ERR) rc = 22;
            for (; rc == 0 && posted < n; ++posted) {
                if (static_cast<int>(qp->rq.size()) >= qp->caps.max_recv_wr) {
                    rc = 12;
                    break;
                }
                qp->rq.push_back(wrs[posted]);
            }
        }
        if (n_posted) *n_posted = posted;
        return rc;
    }

private:
    static Fabric& F() { return Fabric::get(); }
    int            set_state(uint64_t h, LoQp::State from, LoQp::State to, uint32_t dest)
    {
        std::lock_guard<std::mutex> g(F().mu);
        LoQp* qp = reinterpret_cast<LoQp*>(h);
        if (qp->state != from) return 22;
        qp->state = to;
        if (to == LoQp::RTR) qp->dest_qpn = dest;
        return 0;
    }

    std::string name_;
    LinkLayer   link_;
};

class LoProvider final: public VerbsProvider {
public:
    std::string              provider_name() const override { return "loopback"; }
    // two RoCE devices and one InfiniBand device, so that two agents in one process can each have a device (and
    // with it a registry of their own) on the same link type
    std::vector<std::string> list_devices() override { return {"rdma_lo0", "rdma_lo1", "rdma_lo2"}; }
    std::shared_ptr<VerbsDevice> open_device(const std::string& name) override
    {
        if (name == "rdma_lo0" || name == "rdma_lo2") return std::make_shared<LoDevice>(name, LinkLayer::ETHERNET);
        if (name == "rdma_lo1") return std::make_shared<LoDevice>(name, LinkLayer::IB);
        return nullptr;
    }
};

}  // namespace

VerbsProvider* loopback_provider()
{
    static LoProvider p;
    return &p;
}

void loopback_inject_error(WrOp op, int status, int count)
{
    std::lock_guard<std::mutex> g(Fabric::get().mu);
    Fabric::get().injected.push_back(InjectedError{op, status, count});
}

uint64_t loopback_executed_wrs()
{
    return Fabric::get().executed.load();
}

uint64_t loopback_rnr_events()
{
    return Fabric::get().rnr.load();
}

}  // namespace rdma
}  // namespace slime
