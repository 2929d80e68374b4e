#include "transport/rdma/rdma_worker.h"

#include <chrono>
#include <fstream>
#include <pthread.h>
#include <sched.h>
#include <sstream>

#include "core/log.h"
#include "core/nvtx.h"
#include "core/ring.h"
#include "transport/rdma/rdma_endpoint.h"

namespace slime {
namespace rdma {

RdmaWorker::RdmaWorker(int numa_node): numa_(numa_node)
{
    thread_ = std::thread([this] { run(); });
}

RdmaWorker::~RdmaWorker()
{
    stop_.store(true);
    wake();
    if (thread_.joinable()) thread_.join();
}

std::shared_ptr<RdmaWorker> RdmaWorker::for_node(int numa_node)
{
    static std::mutex                                 mu;
    static std::map<int, std::shared_ptr<RdmaWorker>> workers;
    std::lock_guard<std::mutex>                       g(mu);
    auto& w = workers[numa_node];
    if (!w) w = std::make_shared<RdmaWorker>(numa_node);
    return w;
}

void RdmaWorker::add(const std::shared_ptr<RdmaEndpoint>& ep)
{
    {
        std::lock_guard<std::mutex> g(mu_);
        staged_.emplace_back(ep.get(), ep);
        dirty_.store(true, std::memory_order_release);
    }
    wake();
}

void RdmaWorker::remove(const RdmaEndpoint* ep)
{
    std::lock_guard<std::mutex> g(mu_);
    for (auto it = staged_.begin(); it != staged_.end();)
        it = it->first == ep ? staged_.erase(it) : it + 1;
    dirty_.store(true, std::memory_order_release);
}

void RdmaWorker::wake()
{
    if (sleeping_.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> g(mu_);
        cv_.notify_one();
    }
}

// Restrict the thread to the cores of its NUMA node ("0-15,32-47" style list in sysfs).
void RdmaWorker::pin()
{
    if (numa_ < 0) return;
    std::ifstream in("/sys/devices/system/node/node" + std::to_string(numa_) + "/cpulist");
    std::string   list;
    if (!in || !std::getline(in, list)) return;
    cpu_set_t set;
    CPU_ZERO(&set);
    std::stringstream ss(list);
    std::string       item;
    int               n = 0;
    while (std::getline(ss, item, ',')) {
        int lo = 0, hi = 0;
        if (sscanf(item.c_str(), "%d-%d", &lo, &hi) == 2) {
            for (int c = lo; c <= hi && c < CPU_SETSIZE; ++c, ++n) CPU_SET(c, &set);
        }
        else if (sscanf(item.c_str(), "%d", &lo) == 1 && lo < CPU_SETSIZE) {
            CPU_SET(lo, &set);
            ++n;
        }
    }
    if (n > 0 && pthread_setaffinity_np(pthread_self(), sizeof(set), &set) != 0)
        SLIME_LOG_WARN("could not pin the RDMA worker to NUMA node ", numa_);
}

void RdmaWorker::run()
{
    SLIME_NVTX_THREAD("slime.rdma.worker");
    pin();
    std::vector<std::weak_ptr<RdmaEndpoint>> eps;
    int idle = 0;
    while (!stop_.load(std::memory_order_acquire)) {
        if (dirty_.exchange(false, std::memory_order_acq_rel)) {
            std::lock_guard<std::mutex> g(mu_);
            eps.clear();
            for (auto& s : staged_) eps.push_back(s.second);
        }
        int work = 0;
        for (auto& w : eps)
            if (auto ep = w.lock()) work += ep->process();
        loops_.fetch_add(1, std::memory_order_relaxed);
        if (work > 0) {
            idle = 0;
            continue;
        }
        if (++idle < 4000) {
            cpu_pause();
            continue;
        }
        idle = 0;
        sleeps_.fetch_add(1, std::memory_order_relaxed);
        std::unique_lock<std::mutex> g(mu_);
        sleeping_.store(true, std::memory_order_release);
        cv_.wait_for(g, std::chrono::milliseconds(1));
        sleeping_.store(false, std::memory_order_release);
    }
}

}  // namespace rdma
}  // namespace slime
