// The "ibverbs" provider: libibverbs resolved with dlopen / dlsym at first use.
//
// Control-path calls go through the exported symbols; post_send / post_recv / poll_cq /
// req_notify_cq go through the function table of the device context, which is what the library's
// inline wrappers do. Immediate data is converted to network byte order here so that both ends
// see host-order values. Completion events use one completion channel per completion queue:
// req_notify + poll(2) on the channel's descriptor + get/ack event.
//
// This provider cannot be exercised on a host without an RDMA NIC; the layers above it are tested on
// the loopback provider.
#include <arpa/inet.h>
#include <cstring>
#include <dlfcn.h>
#include <fstream>
#include <mutex>
#include <poll.h>

#include "core/env.h"
#include "transport/rdma/ibv_abi.h"
#include "transport/rdma/verbs.h"

namespace slime {
namespace rdma {
namespace {

struct Lib {
    void* handle = nullptr;
    ibv_device** (*get_device_list)(int*)                                   = nullptr;
    void (*free_device_list)(ibv_device**)                                  = nullptr;
    const char* (*get_device_name)(ibv_device*)                             = nullptr;
    ibv_context* (*open_device)(ibv_device*)                                = nullptr;
    int (*close_device)(ibv_context*)                                       = nullptr;
    int (*query_device)(ibv_context*, ibv_device_attr*)                     = nullptr;
    int (*query_port)(ibv_context*, uint8_t, ibv_port_attr*)                = nullptr;
    int (*query_gid)(ibv_context*, uint8_t, int, ibv_gid*)                  = nullptr;
    ibv_pd* (*alloc_pd)(ibv_context*)                                       = nullptr;
    int (*dealloc_pd)(ibv_pd*)                                              = nullptr;
    ibv_mr* (*reg_mr)(ibv_pd*, void*, size_t, int)                          = nullptr;
    int (*dereg_mr)(ibv_mr*)                                                = nullptr;
    ibv_comp_channel* (*create_comp_channel)(ibv_context*)                  = nullptr;
    int (*destroy_comp_channel)(ibv_comp_channel*)                          = nullptr;
    ibv_cq* (*create_cq)(ibv_context*, int, void*, ibv_comp_channel*, int)  = nullptr;
    int (*destroy_cq)(ibv_cq*)                                              = nullptr;
    int (*get_cq_event)(ibv_comp_channel*, ibv_cq**, void**)                = nullptr;
    void (*ack_cq_events)(ibv_cq*, unsigned)                                = nullptr;
    ibv_qp* (*create_qp)(ibv_pd*, ibv_qp_init_attr*)                        = nullptr;
    int (*destroy_qp)(ibv_qp*)                                              = nullptr;
    int (*modify_qp)(ibv_qp*, ibv_qp_attr*, int)                            = nullptr;
    std::string error;

    template<typename F>
    bool sym(F& fn, const char* name)
    {
        fn = reinterpret_cast<F>(dlsym(handle, name));
        if (!fn) error = std::string("libibverbs lacks symbol ") + name;
        return fn != nullptr;
    }

    bool load()
    {
        for (const char* so : {"libibverbs.so.1", "libibverbs.so"}) {
            handle = dlopen(so, RTLD_NOW | RTLD_LOCAL);
            if (handle) break;
        }
        if (!handle) {
            error = "libibverbs could not be loaded (no RDMA user-space stack on this host)";
            return false;
        }
        return sym(get_device_list, "ibv_get_device_list") && sym(free_device_list, "ibv_free_device_list")
               && sym(get_device_name, "ibv_get_device_name") && sym(open_device, "ibv_open_device")
               && sym(close_device, "ibv_close_device") && sym(query_device, "ibv_query_device")
               && sym(query_port, "ibv_query_port") && sym(query_gid, "ibv_query_gid") && sym(alloc_pd, "ibv_alloc_pd")
               && sym(dealloc_pd, "ibv_dealloc_pd") && sym(reg_mr, "ibv_reg_mr") && sym(dereg_mr, "ibv_dereg_mr")
               && sym(create_comp_channel, "ibv_create_comp_channel") && sym(destroy_comp_channel, "ibv_destroy_comp_channel")
               && sym(create_cq, "ibv_create_cq") && sym(destroy_cq, "ibv_destroy_cq") && sym(get_cq_event, "ibv_get_cq_event")
               && sym(ack_cq_events, "ibv_ack_cq_events") && sym(create_qp, "ibv_create_qp") && sym(destroy_qp, "ibv_destroy_qp")
               && sym(modify_qp, "ibv_modify_qp");
    }
};

Lib& lib()
{
    static Lib  l;
    static bool once = (l.load(), true);
    (void)once;
    return l;
}

struct CqBox {
    ibv_cq*           cq      = nullptr;
    ibv_comp_channel* channel = nullptr;
};

class IbvDevice final: public VerbsDevice {
public:
    IbvDevice(std::string name, ibv_context* ctx): name_(std::move(name)), ctx_(ctx) {}
    ~IbvDevice() override
    {
        if (ctx_) lib().close_device(ctx_);
    }

    std::string name() const override { return name_; }

    DeviceAttr query_device() override
    {
        ibv_device_attr a;
        memset(&a, 0, sizeof(a));
        DeviceAttr out;
        if (lib().query_device(ctx_, &a) == 0) {
            out.max_cqe        = a.max_cqe;
            out.max_qp_wr      = a.max_qp_wr;
            out.max_sge        = a.max_sge;
            out.max_qp_rd_atom = a.max_qp_rd_atom;
            out.phys_port_cnt  = a.phys_port_cnt;
        }
        return out;
    }

    PortAttr query_port(int port) override
    {
        ibv_port_attr a;
        memset(&a, 0, sizeof(a));
        PortAttr out;
        if (lib().query_port(ctx_, static_cast<uint8_t>(port), &a) == 0) {
            out.active      = a.state == IBV_PORT_ACTIVE;
            out.lid         = a.lid;
            out.active_mtu  = a.active_mtu;
            out.gid_tbl_len = a.gid_tbl_len;
            out.link_layer  = a.link_layer == IBV_LINK_LAYER_ETHERNET ? LinkLayer::ETHERNET
                                                                       : (a.link_layer == IBV_LINK_LAYER_INFINIBAND ? LinkLayer::IB : LinkLayer::UNKNOWN);
        }
        return out;
    }

    bool query_gid(int port, int index, Gid& out) override
    {
        ibv_gid g;
        if (lib().query_gid(ctx_, static_cast<uint8_t>(port), index, &g) != 0) return false;
        memcpy(out.data(), g.raw, 16);
        return true;
    }

    int find_roce_v2_gid(int port, int gid_tbl_len) override
    {
        // sysfs names the protocol of every table entry; prefer an IPv4-mapped RoCE v2 address
        int any_v2 = -1;
        for (int i = 0; i < gid_tbl_len; ++i) {
            std::ifstream in("/sys/class/infiniband/" + name_ + "/ports/" + std::to_string(port) + "/gid_attrs/types/" + std::to_string(i));
            std::string   type;
            if (!in || !std::getline(in, type)) continue;
            if (type.find("v2") == std::string::npos) continue;
            Gid g;
            if (!query_gid(port, i, g)) continue;
            bool zero = true;
            for (uint8_t b : g) zero = zero && b == 0;
            if (zero) continue;
            if (any_v2 < 0) any_v2 = i;
            bool mapped = g[10] == 0xff && g[11] == 0xff;
            for (int k = 0; k < 10; ++k) mapped = mapped && g[k] == 0;
            if (mapped) return i;
        }
        return any_v2;
    }

    uint64_t alloc_pd() override { return reinterpret_cast<uint64_t>(lib().alloc_pd(ctx_)); }
    void     dealloc_pd(uint64_t pd) override
    {
        if (pd) lib().dealloc_pd(reinterpret_cast<ibv_pd*>(pd));
    }

    bool reg_mr(uint64_t pd, uintptr_t addr, uint64_t len, MrKeys& out) override
    {
        ibv_mr* mr = lib().reg_mr(reinterpret_cast<ibv_pd*>(pd), reinterpret_cast<void*>(addr), len,
                                  IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ);
        if (!mr) return false;
        out.handle = reinterpret_cast<uint64_t>(mr);
        out.lkey   = mr->lkey;
        out.rkey   = mr->rkey;
        return true;
    }
    void dereg_mr(uint64_t h) override
    {
        if (h) lib().dereg_mr(reinterpret_cast<ibv_mr*>(h));
    }

    uint64_t create_cq(int depth) override
    {
        auto* box    = new CqBox();
        box->channel = lib().create_comp_channel(ctx_);
        box->cq      = lib().create_cq(ctx_, depth, nullptr, box->channel, 0);
        if (!box->cq) {
            if (box->channel) lib().destroy_comp_channel(box->channel);
            delete box;
            return 0;
        }
        return reinterpret_cast<uint64_t>(box);
    }
    void destroy_cq(uint64_t h) override
    {
        auto* box = reinterpret_cast<CqBox*>(h);
        if (!box) return;
        lib().destroy_cq(box->cq);
        if (box->channel) lib().destroy_comp_channel(box->channel);
        delete box;
    }
    int poll_cq(uint64_t h, int max_entries, Completion* out) override
    {
        auto*  box = reinterpret_cast<CqBox*>(h);
        ibv_wc wc[64];
        int    total = 0;
        while (total < max_entries) {
            const int want = std::min(max_entries - total, 64);
            const int n    = ctx_->ops.poll_cq(box->cq, want, wc);
            if (n <= 0) break;
            for (int i = 0; i < n; ++i) {
                Completion& c = out[total++];
                c.wr_id       = wc[i].wr_id;
                c.status      = wc[i].status;
                c.op          = static_cast<WcOp>(wc[i].opcode);
                c.has_imm     = (wc[i].wc_flags & IBV_WC_WITH_IMM) != 0;
                c.imm         = ntohl(wc[i].imm_data);
                c.byte_len    = wc[i].byte_len;
                c.qp_num      = wc[i].qp_num;
            }
            if (n < want) break;
        }
        return total;
    }
    bool wait_cq_event(uint64_t h, int timeout_ms) override
    {
        auto* box = reinterpret_cast<CqBox*>(h);
        if (!box->channel) return false;
        if (ctx_->ops.req_notify_cq(box->cq, 0) != 0) return false;
        pollfd pfd{box->channel->fd, POLLIN, 0};
        if (::poll(&pfd, 1, timeout_ms) <= 0) return false;
        ibv_cq* ev_cq  = nullptr;
        void*   ev_ctx = nullptr;
        if (lib().get_cq_event(box->channel, &ev_cq, &ev_ctx) != 0) return false;
        lib().ack_cq_events(ev_cq, 1);
        return true;
    }

    uint64_t create_qp(uint64_t pd, uint64_t cq, const QpCaps& caps, uint32_t& qp_num_out) override
    {
        auto*            box = reinterpret_cast<CqBox*>(cq);
        ibv_qp_init_attr a;
        memset(&a, 0, sizeof(a));
        a.send_cq             = box->cq;
        a.recv_cq             = box->cq;
        a.qp_type             = IBV_QPT_RC;
        a.cap.max_send_wr     = caps.max_send_wr;
        a.cap.max_recv_wr     = caps.max_recv_wr;
        a.cap.max_send_sge    = 1;
        a.cap.max_recv_sge    = 1;
        a.cap.max_inline_data = caps.max_inline;
        ibv_qp* qp            = lib().create_qp(reinterpret_cast<ibv_pd*>(pd), &a);
        if (!qp) return 0;
        qp_num_out = qp->qp_num;
        return reinterpret_cast<uint64_t>(qp);
    }
    void destroy_qp(uint64_t qp) override
    {
        if (qp) lib().destroy_qp(reinterpret_cast<ibv_qp*>(qp));
    }

    int qp_to_init(uint64_t qp, int port) override
    {
        ibv_qp_attr a;
        memset(&a, 0, sizeof(a));
        a.qp_state        = IBV_QPS_INIT;
        a.port_num        = static_cast<uint8_t>(port);
        a.pkey_index      = 0;
        a.qp_access_flags = IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ;
        return lib().modify_qp(reinterpret_cast<ibv_qp*>(qp), &a, IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS);
    }
    int qp_to_rtr(uint64_t qp, const QpRoute& r) override
    {
        ibv_qp_attr a;
        memset(&a, 0, sizeof(a));
        a.qp_state           = IBV_QPS_RTR;
        a.path_mtu           = r.mtu;
        a.dest_qp_num        = r.dest_qpn;
        a.rq_psn             = r.dest_psn;
        a.max_dest_rd_atomic = static_cast<uint8_t>(r.max_dest_rd_atomic);
        a.min_rnr_timer      = static_cast<uint8_t>(r.min_rnr_timer);
        a.ah_attr.port_num   = static_cast<uint8_t>(r.port);
        a.ah_attr.sl         = static_cast<uint8_t>(r.service_level);
        a.ah_attr.dlid       = r.dest_lid;
        if (r.is_global) {
            a.ah_attr.is_global      = 1;
            a.ah_attr.grh.hop_limit  = 64;
            a.ah_attr.grh.sgid_index = static_cast<uint8_t>(r.sgid_index);
            memcpy(a.ah_attr.grh.dgid.raw, r.dest_gid.data(), 16);
        }
        return lib().modify_qp(reinterpret_cast<ibv_qp*>(qp), &a,
                               IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN
                                   | IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER);
    }
    int qp_to_rts(uint64_t qp, const QpRoute& r) override
    {
        ibv_qp_attr a;
        memset(&a, 0, sizeof(a));
        a.qp_state      = IBV_QPS_RTS;
        a.timeout       = static_cast<uint8_t>(r.timeout);
        a.retry_cnt     = static_cast<uint8_t>(r.retry_cnt);
        a.rnr_retry     = static_cast<uint8_t>(r.rnr_retry);
        a.sq_psn        = r.local_psn;
        a.max_rd_atomic = static_cast<uint8_t>(r.max_rd_atomic);
        return lib().modify_qp(reinterpret_cast<ibv_qp*>(qp), &a,
                               IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN | IBV_QP_MAX_QP_RD_ATOMIC);
    }

    int post_send(uint64_t qp, const SendWr* wrs, int n, int* n_posted) override
    {
        // chains of up to 64 work requests built on the stack
        int done = 0, rc = 0;
        while (done < n && rc == 0) {
            ibv_send_wr chain[64];
            ibv_sge     sges[64];
            const int   m = std::min(n - done, 64);
            for (int i = 0; i < m; ++i) {
                const SendWr& w = wrs[done + i];
                memset(&chain[i], 0, sizeof(ibv_send_wr));
                sges[i]             = ibv_sge{w.sge.addr, w.sge.length, w.sge.lkey};
                chain[i].wr_id      = w.wr_id;
                chain[i].next       = i + 1 < m ? &chain[i + 1] : nullptr;
                chain[i].sg_list    = &sges[i];
                chain[i].num_sge    = 1;
                chain[i].opcode     = static_cast<int>(w.op);
                chain[i].send_flags = (w.signaled ? IBV_SEND_SIGNALED : 0) | (w.inline_data ? IBV_SEND_INLINE : 0);
                chain[i].imm_data   = htonl(w.imm);
                chain[i].wr.rdma.remote_addr = w.remote_addr;
                chain[i].wr.rdma.rkey        = w.rkey;
            }
            ibv_send_wr* bad = nullptr;
            rc               = ctx_->ops.post_send(reinterpret_cast<ibv_qp*>(qp), chain, &bad);
            done += (rc == 0 || bad == nullptr) ? (rc == 0 ? m : 0) : static_cast<int>(bad - chain);
        }
        if (n_posted) *n_posted = done;
        return rc;
    }
    int post_recv(uint64_t qp, const RecvWr* wrs, int n, int* n_posted) override
    {
        int done = 0, rc = 0;
        while (done < n && rc == 0) {
            ibv_recv_wr chain[64];
            ibv_sge     sges[64];
            const int   m = std::min(n - done, 64);
            for (int i = 0; i < m; ++i) {
                const RecvWr& w  = wrs[done + i];
                sges[i]          = ibv_sge{w.sge.addr, w.sge.length, w.sge.lkey};
                chain[i].wr_id   = w.wr_id;
                chain[i].next    = i + 1 < m ? &chain[i + 1] : nullptr;
                chain[i].sg_list = w.sge.length ? &sges[i] : nullptr;
                chain[i].num_sge = w.sge.length ? 1 : 0;
            }
            ibv_recv_wr* bad = nullptr;
            rc               = ctx_->ops.post_recv(reinterpret_cast<ibv_qp*>(qp), chain, &bad);
            done += (rc == 0 || bad == nullptr) ? (rc == 0 ? m : 0) : static_cast<int>(bad - chain);
        }
        if (n_posted) *n_posted = done;
        return rc;
    }

private:
    std::string  name_;
    ibv_context* ctx_;
};

class IbvProvider final: public VerbsProvider {
public:
    std::string provider_name() const override { return "ibverbs"; }

    std::vector<std::string> list_devices() override
    {
        std::vector<std::string> out;
        int                      n    = 0;
        ibv_device**             list = lib().get_device_list(&n);
        if (!list) return out;
        for (int i = 0; i < n; ++i) out.emplace_back(lib().get_device_name(list[i]));
        lib().free_device_list(list);
        return out;
    }

    std::shared_ptr<VerbsDevice> open_device(const std::string& name) override
    {
        int          n    = 0;
        ibv_device** list = lib().get_device_list(&n);
        if (!list) return nullptr;
        std::shared_ptr<VerbsDevice> out;
        for (int i = 0; i < n && !out; ++i) {
            if (name == lib().get_device_name(list[i])) {
                if (ibv_context* ctx = lib().open_device(list[i])) out = std::make_shared<IbvDevice>(name, ctx);
            }
        }
        lib().free_device_list(list);
        return out;
    }
};

}  // namespace

VerbsProvider* ibverbs_provider(std::string* why)
{
    Lib& l = lib();
    if (!l.handle || !l.error.empty()) {
        if (why) *why = l.error;
        return nullptr;
    }
    static IbvProvider p;
    return &p;
}

VerbsProvider* default_provider(std::string* why)
{
    const std::string pick = get_env<std::string>("SLIME_RDMA_PROVIDER", "");
    if (pick == "loopback") return loopback_provider();
    std::string    reason;
    VerbsProvider* p = ibverbs_provider(&reason);
    if (p && p->list_devices().empty()) {
        reason = "libibverbs loaded but reports no RDMA device";
        p      = nullptr;
    }
    if (!p && why) *why = reason;
    return p;
}

}  // namespace rdma
}  // namespace slime
