// One opened RDMA device port: protection domain, one completion queue, the completion thread,
// the address this side advertises, and a memory pool whose registrations carry the device's keys.
//
// Completions are routed by queue-pair number to a CompletionSink (an endpoint) held weakly, so an
// endpoint may go away while late flush completions are still in the queue. The completion thread is
// adaptive: it polls in bursts, and after a long run of empty polls arms the queue and sleeps on the
// completion event with a 100 ms limit. One context exists per (provider, device, port), shared by
// every endpoint on that port (ContextManager).
//
// Role in the reference: RDMAContext, its cq_poll_handle thread and GlobalContextManager
// (dlslime/csrc/engine/rdma/rdma_context.cpp:51-317, rdma_context_pool.h:15-75 in the reference).
#pragma once

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <string>
#include <thread>
#include <unordered_map>

#include "core/json.hpp"
#include "engine/memory_pool.h"
#include "transport/rdma/verbs.h"

namespace slime {
namespace rdma {

class CompletionSink {
public:
    virtual ~CompletionSink()                        = default;
    virtual void on_completion(const Completion& wc) = 0;
};

// What one queue pair tells its peer.
struct QpInfo {
    uint32_t qpn  = 0;
    uint32_t psn  = 0;
    Gid      gid{};
    int      gidx = 0;
    uint16_t lid  = 0;
    int      mtu  = 3;

    Json          to_json() const;
    static QpInfo from_json(const Json& j);
};

class RdmaContext: public std::enable_shared_from_this<RdmaContext> {
public:
    // link_type: "RoCE" | "IB" | "" (accept what the port has). Throws std::runtime_error with the reason.
    RdmaContext(VerbsProvider* provider, const std::string& device, int port, const std::string& link_type);
    ~RdmaContext();

    const std::string& device_name() const { return device_name_; }
    int                port() const { return port_; }
    bool               is_roce() const { return port_attr_.link_layer == LinkLayer::ETHERNET; }
    const Gid&         gid() const { return gid_; }
    int                gid_index() const { return gid_index_; }
    uint16_t           lid() const { return port_attr_.lid; }
    int                mtu() const { return port_attr_.active_mtu; }
    int                max_qp_wr() const { return dev_attr_.max_qp_wr; }
    int                obs_link() const { return obs_link_; }
    int                numa_node() const { return numa_node_; }
    VerbsDevice&       dev() { return *dev_; }
    uint64_t           pd() const { return pd_; }
    uint64_t           cq() const { return cq_; }

    // A pool whose register / unregister hooks call reg_mr / dereg_mr on this context's domain.
    std::shared_ptr<LocalMemoryPool> make_pool();
    // The pool shared by every endpoint of this context: a region has one handle and one key per device,
    // whichever endpoint registered it (a key is valid on every queue pair of the protection domain).
    std::shared_ptr<LocalMemoryPool> shared_pool();

    void add_sink(uint32_t qp_num, const std::shared_ptr<CompletionSink>& sink);
    void remove_sink(uint32_t qp_num);

    uint64_t completions_seen() const { return completions_.load(); }
    uint64_t cq_sleeps() const { return sleeps_.load(); }

private:
    void cq_loop();

    VerbsProvider*               provider_;
    std::shared_ptr<VerbsDevice> dev_;
    std::string                  device_name_;
    int                          port_ = 1;
    DeviceAttr                   dev_attr_;
    PortAttr                     port_attr_;
    Gid                          gid_{};
    int                          gid_index_ = 0;
    uint64_t                     pd_ = 0, cq_ = 0;
    int                          obs_link_  = -1;
    int                          numa_node_ = -1;

    std::shared_mutex                                          sinks_mu_;
    std::unordered_map<uint32_t, std::weak_ptr<CompletionSink>> sinks_;

    std::atomic<bool>     stop_{false};
    std::atomic<uint64_t> completions_{0}, sleeps_{0};
    std::thread           cq_thread_;
    std::mutex                       pool_mu_;
    std::shared_ptr<LocalMemoryPool> shared_pool_;
};

class ContextManager {
public:
    static ContextManager& get();
    // device "" picks the first device of the provider (and any failure to open a named device falls
    // back to the first one, as the reference does).
    std::shared_ptr<RdmaContext> acquire(const std::string& device, int port, const std::string& link_type);
    void                         clear();  // drops every cached context (tests)

private:
    std::mutex                                          mu_;
    std::map<std::string, std::shared_ptr<RdmaContext>> contexts_;
};

}  // namespace rdma
}  // namespace slime
