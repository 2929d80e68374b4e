// Progress threads of the RDMA endpoints: one per NUMA node, pinned to that node's cores, looping
// over its endpoints' process(). A worker that found nothing to do for a while sleeps on a condition
// variable (1 ms limit) and is woken by submissions and by completions that unblock queued work, so an
// idle process burns no core. Endpoints are held weakly; adding and removing goes through a staging
// list so the hot loop takes no lock.
//
// Role in the reference: RDMAWorker / GlobalWorkerManager
// (dlslime/csrc/engine/rdma/rdma_worker.cpp:40-117, rdma_worker_pool.h:17-28 in the reference), which
// busy-loop without sleeping.
#pragma once

#include <atomic>
#include <condition_variable>
#include <map>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

namespace slime {
namespace rdma {

class RdmaEndpoint;

class RdmaWorker {
public:
    explicit RdmaWorker(int numa_node);
    ~RdmaWorker();

    void add(const std::shared_ptr<RdmaEndpoint>& ep);
    void remove(const RdmaEndpoint* ep);
    void wake();

    int      numa_node() const { return numa_; }
    uint64_t loops() const { return loops_.load(); }
    uint64_t sleeps() const { return sleeps_.load(); }

    // One worker per NUMA node (node -1 = unpinned), created on first use.
    static std::shared_ptr<RdmaWorker> for_node(int numa_node);

private:
    void run();
    void pin();

    int                     numa_;
    std::atomic<bool>       stop_{false}, dirty_{false}, sleeping_{false};
    std::atomic<uint64_t>   loops_{0}, sleeps_{0};
    std::mutex              mu_;
    std::condition_variable cv_;
    std::vector<std::pair<const RdmaEndpoint*, std::weak_ptr<RdmaEndpoint>>> staged_;
    std::thread             thread_;
};

}  // namespace rdma
}  // namespace slime
