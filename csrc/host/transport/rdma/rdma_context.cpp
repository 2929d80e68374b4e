#include "transport/rdma/rdma_context.h"

#include <chrono>
#include <cstdio>
#include <stdexcept>

#include "core/env.h"
#include "core/log.h"
#include "core/nvtx.h"
#include "core/ring.h"
#include "obs/obs.h"
#include "topology/topology.h"

namespace slime {
namespace rdma {

Json QpInfo::to_json() const
{
    Json j    = Json::object();
    j["qpn"]  = static_cast<long long>(qpn);
    j["psn"]  = static_cast<long long>(psn);
    j["gidx"] = gidx;
    j["lid"]  = static_cast<long long>(lid);
    j["mtu"]  = mtu;
    char hex[33];
    for (int i = 0; i < 16; ++i) snprintf(hex + 2 * i, 3, "%02x", gid[i]);
    j["gid"] = std::string(hex, 32);
    return j;
}

QpInfo QpInfo::from_json(const Json& j)
{
    QpInfo q;
    q.qpn  = static_cast<uint32_t>(j["qpn"].as_int());
    q.psn  = static_cast<uint32_t>(j["psn"].as_int());
    q.gidx = static_cast<int>(j["gidx"].as_int());
    q.lid  = static_cast<uint16_t>(j["lid"].as_int());
    q.mtu  = static_cast<int>(j["mtu"].as_int());
    const std::string hex = j["gid"].string_or("");
    for (int i = 0; i < 16 && 2 * i + 1 < static_cast<int>(hex.size()); ++i)
        q.gid[i] = static_cast<uint8_t>(std::stoi(hex.substr(2 * i, 2), nullptr, 16));
    return q;
}

RdmaContext::RdmaContext(VerbsProvider* provider, const std::string& device, int port, const std::string& link_type):
    provider_(provider), port_(port)
{
    const auto devices = provider->list_devices();
    if (devices.empty()) throw std::runtime_error("RDMA provider " + provider->provider_name() + " has no device");
    std::string pick = device;
    if (!pick.empty()) dev_ = provider->open_device(pick);
    if (!dev_) {
        if (!pick.empty()) SLIME_LOG_WARN("RDMA device ", pick, " could not be opened; falling back to ", devices[0]);
        pick = devices[0];
        dev_ = provider->open_device(pick);
    }
    if (!dev_) throw std::runtime_error("cannot open RDMA device " + pick);
    device_name_ = pick;
    dev_attr_    = dev_->query_device();
    port_attr_   = dev_->query_port(port);
    if (!port_attr_.active) throw std::runtime_error("port " + std::to_string(port) + " of " + pick + " is not active");
    const std::string want = topology::normalize_link_type(link_type);
    if (!link_type.empty()) {
        const bool roce = port_attr_.link_layer == LinkLayer::ETHERNET;
        if ((want == "RoCE" && !roce) || (want == "IB" && roce))
            throw std::runtime_error("port " + std::to_string(port) + " of " + pick + " is " + (roce ? "RoCE" : "IB") + ", not " + want);
    }
    const int forced = engine_env().gid_index;
    if (forced >= 0) {
        gid_index_ = forced;
    }
    else if (is_roce()) {
        gid_index_ = dev_->find_roce_v2_gid(port, port_attr_.gid_tbl_len);
        if (gid_index_ < 0) throw std::runtime_error("no RoCE v2 GID on " + pick + " (set SLIME_GID_INDEX)");
    }
    if (!dev_->query_gid(port, gid_index_, gid_)) throw std::runtime_error("cannot read GID " + std::to_string(gid_index_) + " of " + pick);

    pd_ = dev_->alloc_pd();
    if (!pd_) throw std::runtime_error("cannot allocate a protection domain on " + pick);
    int depth = engine_env().max_cq_depth;
    if (dev_attr_.max_cqe > 0 && depth > dev_attr_.max_cqe) depth = dev_attr_.max_cqe;
    cq_ = dev_->create_cq(depth);
    if (!cq_) {
        dev_->dealloc_pd(pd_);
        throw std::runtime_error("cannot create a completion queue on " + pick);
    }
    obs_link_  = obs::register_link(pick, "rdma");
    numa_node_ = topology::numa_node_of(pick);
    cq_thread_ = std::thread([this] { cq_loop(); });
}

RdmaContext::~RdmaContext()
{
    stop_.store(true);
    if (cq_thread_.joinable()) cq_thread_.join();
    if (cq_) dev_->destroy_cq(cq_);
    if (pd_) dev_->dealloc_pd(pd_);
}

std::shared_ptr<LocalMemoryPool> RdmaContext::make_pool()
{
    auto pool = std::make_shared<LocalMemoryPool>();
    // Weak: the shared pool is owned by the context itself. A pool that outlives its context cannot register.
    std::weak_ptr<RdmaContext> weak = shared_from_this();
    pool->on_register = [weak](MemoryRegion& r) {
        auto self = weak.lock();
        if (!self) throw std::runtime_error("the RDMA context of this memory pool is gone");
        MrKeys k;
        if (!self->dev_->reg_mr(self->pd_, r.addr, r.length, k))
            throw std::runtime_error("memory registration of " + std::to_string(r.length) + " bytes failed on " + self->device_name_);
        r.lkey   = k.lkey;
        r.rkey   = k.rkey;
        r.opaque = k.handle;
    };
    pool->on_unregister = [weak](const MemoryRegion& r) {
        auto self = weak.lock();
        if (self && r.opaque) self->dev_->dereg_mr(r.opaque);
    };
    return pool;
}

std::shared_ptr<LocalMemoryPool> RdmaContext::shared_pool()
{
    std::lock_guard<std::mutex> g(pool_mu_);
    if (!shared_pool_) shared_pool_ = make_pool();
    return shared_pool_;
}

void RdmaContext::add_sink(uint32_t qp_num, const std::shared_ptr<CompletionSink>& sink)
{
    std::unique_lock<std::shared_mutex> g(sinks_mu_);
    sinks_[qp_num] = sink;
}

void RdmaContext::remove_sink(uint32_t qp_num)
{
    std::unique_lock<std::shared_mutex> g(sinks_mu_);
    sinks_.erase(qp_num);
}

void RdmaContext::cq_loop()
{
    SLIME_NVTX_THREAD("slime.rdma.cq");
    const int               burst = std::max(1, engine_env().poll_count);
    std::vector<Completion> wcs(burst);
    int                     empty_spins = 0;
    // One-entry cache: completions come in runs for the same queue pair.
    uint32_t                        cached_qpn = 0;
    std::shared_ptr<CompletionSink> cached;
    while (!stop_.load(std::memory_order_acquire)) {
        const int n = dev_->poll_cq(cq_, burst, wcs.data());
        if (n <= 0) {
            cached.reset();
            cached_qpn = 0;
            if (++empty_spins < 10000) {
                cpu_pause();
                continue;
            }
            empty_spins = 0;
            sleeps_.fetch_add(1, std::memory_order_relaxed);
            dev_->wait_cq_event(cq_, 100);
            continue;
        }
        empty_spins = 0;
        completions_.fetch_add(n, std::memory_order_relaxed);
        for (int i = 0; i < n; ++i) {
            const Completion& wc = wcs[i];
            if (wc.status != WC_SUCCESS && wc.status != WC_WR_FLUSH_ERR) {
                SLIME_LOG_WARN("completion error ", wc.status, " on ", device_name_, " qp ", wc.qp_num);
                obs::record_cq_error(obs_link_);
            }
            if (wc.qp_num != cached_qpn || !cached) {
                std::shared_lock<std::shared_mutex> g(sinks_mu_);
                auto it    = sinks_.find(wc.qp_num);
                cached     = it == sinks_.end() ? nullptr : it->second.lock();
                cached_qpn = wc.qp_num;
            }
            if (cached) cached->on_completion(wc);
        }
    }
}

ContextManager& ContextManager::get()
{
    static ContextManager m;
    return m;
}

std::shared_ptr<RdmaContext> ContextManager::acquire(const std::string& device, int port, const std::string& link_type)
{
    std::string    why;
    VerbsProvider* provider = default_provider(&why);
    if (!provider) throw std::runtime_error("no RDMA provider: " + why);
    std::lock_guard<std::mutex> g(mu_);
    const std::string key = provider->provider_name() + "/" + device + "/" + std::to_string(port);
    auto it = contexts_.find(key);
    if (it != contexts_.end()) return it->second;
    auto ctx = std::make_shared<RdmaContext>(provider, device, port, link_type);
    contexts_[key] = ctx;
    // a fallback to another device must not be created twice under its real name
    const std::string real = provider->provider_name() + "/" + ctx->device_name() + "/" + std::to_string(port);
    auto rit = contexts_.find(real);
    if (rit == contexts_.end()) contexts_[real] = ctx;
    return ctx;
}

void ContextManager::clear()
{
    std::lock_guard<std::mutex> g(mu_);
    contexts_.clear();
}

}  // namespace rdma
}  // namespace slime
