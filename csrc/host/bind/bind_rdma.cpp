// Bindings of the RDMA transport: the endpoint, its context, and the provider controls.
#include "bind/bind_common.h"
#include "transport/rdma/rdma_endpoint.h"
#include "transport/rdma/rdma_worker.h"

using namespace slime;
using namespace slime::rdma;

namespace {

// `RDMAMemoryPool(context)` of the reference's API (dlslime/csrc/python/bind.cpp:163-189 in the reference). Regions
// are registered once per device here, so the object is a view of the context's pool rather than a pool of its own:
// two views of one context see the same regions.
struct RdmaPoolView {
    std::shared_ptr<RdmaContext>     ctx;
    std::shared_ptr<LocalMemoryPool> pool;
    explicit RdmaPoolView(std::shared_ptr<RdmaContext> c): ctx(std::move(c))
    {
        if (!ctx) throw std::runtime_error("RDMAMemoryPool needs a context");
        pool = ctx->shared_pool();
    }
};

// `RDMAWorker(dev_name | socket_id, id)` of the reference's API (bind.cpp:272-280 in the reference): a progress
// thread of the caller's own. Endpoints are progressed by a shared per-NUMA-node worker unless they are given one
// of these; `start()` creates the thread, `stop()` ends it and hands its endpoints back to the shared workers.
struct RdmaWorkerHandle {
    int                                      numa = -1;
    int                                      id   = 0;
    std::shared_ptr<RdmaWorker>              worker;
    std::vector<std::weak_ptr<RdmaEndpoint>> eps;
    std::mutex                               mu;

    void start()
    {
        std::lock_guard<std::mutex> g(mu);
        if (worker) return;
        worker = std::make_shared<RdmaWorker>(numa);
        for (auto& w : eps)
            if (auto ep = w.lock()) ep->set_worker(worker);
    }
    void stop()
    {
        std::lock_guard<std::mutex> g(mu);
        if (!worker) return;
        for (auto& w : eps)
            if (auto ep = w.lock()) ep->set_worker(nullptr);
        worker.reset();
    }
    int add_endpoint(const std::shared_ptr<RdmaEndpoint>& ep)
    {
        if (!ep) throw std::runtime_error("RDMAWorker.add_endpoint: no endpoint");
        std::lock_guard<std::mutex> g(mu);
        eps.push_back(ep);
        if (worker) ep->set_worker(worker);
        return static_cast<int>(eps.size()) - 1;
    }
    ~RdmaWorkerHandle() { stop(); }
};

std::shared_ptr<RdmaEndpoint> make_endpoint(std::shared_ptr<RdmaContext> ctx, int num_qp, const std::shared_ptr<RdmaWorkerHandle>& wh)
{
    auto ep = RdmaEndpoint::create(std::move(ctx), num_qp, nullptr);
    if (wh) wh->add_endpoint(ep);
    return ep;
}

}  // namespace

void bind_rdma(py::module_& m)
{
    py::class_<RdmaContext, std::shared_ptr<RdmaContext>>(m, "RDMAContext")
        .def_static(
            "acquire", [](const std::string& dev, int port, const std::string& link) { return ContextManager::get().acquire(dev, port, link); },
            py::arg("device") = "", py::arg("ib_port") = 1, py::arg("link_type") = "")
        .def("device_name", &RdmaContext::device_name)
        .def("port", &RdmaContext::port)
        .def("link_type", [](RdmaContext& c) { return std::string(c.is_roce() ? "RoCE" : "IB"); })
        .def("gid_index", &RdmaContext::gid_index)
        .def("lid", &RdmaContext::lid)
        .def("mtu", &RdmaContext::mtu)
        .def("numa_node", &RdmaContext::numa_node)
        .def("completions_seen", &RdmaContext::completions_seen)
        .def("cq_sleeps", &RdmaContext::cq_sleeps);

    py::class_<RdmaPoolView, std::shared_ptr<RdmaPoolView>>(m, "RDMAMemoryPool")
        .def(py::init<std::shared_ptr<RdmaContext>>(), py::arg("context"))
        .def("register_memory_region",
             [](RdmaPoolView& v, uintptr_t ptr, uint64_t length, std::optional<std::string> name) {
                 return v.pool->register_memory_region(ptr, length, name);
             },
             py::arg("data_ptr"), py::arg("length"), py::arg("name") = py::none())
        .def("get_handle", [](RdmaPoolView& v, const std::string& name) { return v.pool->get_mr_handle(name); })
        .def("unregister_memory_region",
             [](RdmaPoolView& v, py::object key) {
                 if (py::isinstance<py::str>(key)) return v.pool->unregister_memory_region(key.cast<std::string>());
                 return v.pool->unregister_memory_region(key.cast<int32_t>());
             },
             py::arg("key"))
        .def("mr_info", [](RdmaPoolView& v) { return v.pool->mr_info(); })
        .def("context", [](RdmaPoolView& v) { return v.ctx; });

    // declared before the endpoint (whose constructors take one), filled in after it (add_endpoint takes an endpoint)
    py::class_<RdmaWorkerHandle, std::shared_ptr<RdmaWorkerHandle>> worker_cls(m, "RDMAWorker");

    // The three constructor forms of the reference (bind.cpp:191-204 in the reference): from a pool, from a context,
    // from a device name. `worker` = an RDMAWorker of the caller, or None for the shared per-node worker.
    py::class_<RdmaEndpoint, Endpoint, std::shared_ptr<RdmaEndpoint>>(m, "RDMAEndpoint")
        .def(py::init([](std::shared_ptr<RdmaPoolView> pool, int num_qp, std::shared_ptr<RdmaWorkerHandle> worker) {
                 if (!pool) throw std::runtime_error("RDMAEndpoint: pool is None");
                 return make_endpoint(pool->ctx, num_qp, worker);
             }),
             py::arg("pool"), py::arg("num_qp") = 1, py::arg("worker") = nullptr)
        .def(py::init([](std::shared_ptr<RdmaContext> ctx, int num_qp, std::shared_ptr<RdmaWorkerHandle> worker) {
                 return make_endpoint(std::move(ctx), num_qp, worker);
             }),
             py::arg("context"), py::arg("num_qp") = 1, py::arg("worker") = nullptr)
        .def(py::init([](const std::string& dev, int port, const std::string& link, int num_qp, std::shared_ptr<RdmaWorkerHandle> worker) {
                 return make_endpoint(ContextManager::get().acquire(dev, port, link), num_qp, worker);
             }),
             py::arg("device_name") = "", py::arg("ib_port") = 1, py::arg("link_type") = "", py::arg("num_qp") = 0,
             py::arg("worker") = nullptr)
        .def("get_pool", [](RdmaEndpoint& ep) { return std::make_shared<RdmaPoolView>(ep.context()); })
        .def("num_qp", &RdmaEndpoint::num_qp)
        .def("context", &RdmaEndpoint::context)
        .def("process", &RdmaEndpoint::process)
        .def("cancel_all", &RdmaEndpoint::cancel_all, py::call_guard<py::gil_scoped_release>())
        .def("posted_wrs", &RdmaEndpoint::posted_wrs)
        .def("signaled_wrs", &RdmaEndpoint::signaled_wrs)
        .def("credit_stalls", &RdmaEndpoint::credit_stalls);

    worker_cls
        .def(py::init([](const std::string& dev_name, int id) {
                 auto w = std::make_shared<RdmaWorkerHandle>();
                 w->id  = id;
                 try {
                     w->numa = ContextManager::get().acquire(dev_name, 1, "")->numa_node();
                 }
                 catch (const std::exception&) {
                     w->numa = -1;  // no such device here: an unpinned thread
                 }
                 return w;
             }),
             py::arg("dev_name"), py::arg("id"))
        .def(py::init([](int32_t socket_id, int id) {
                 auto w  = std::make_shared<RdmaWorkerHandle>();
                 w->id   = id;
                 w->numa = socket_id;
                 return w;
             }),
             py::arg("socket_id"), py::arg("id"))
        .def("start", &RdmaWorkerHandle::start)
        .def("stop", &RdmaWorkerHandle::stop, py::call_guard<py::gil_scoped_release>())
        .def("add_endpoint", &RdmaWorkerHandle::add_endpoint, py::arg("endpoint"))
        .def("running", [](RdmaWorkerHandle& w) { return w.worker != nullptr; })
        .def("numa_node", [](RdmaWorkerHandle& w) { return w.numa; })
        .def("stats", [](RdmaWorkerHandle& w) {
            py::dict d;
            d["loops"]  = w.worker ? w.worker->loops() : 0;
            d["sleeps"] = w.worker ? w.worker->sleeps() : 0;
            return d;
        });


    // Which verbs provider new contexts would use: (name, "") or (None, reason).
    m.def("rdma_provider", []() -> py::tuple {
        std::string    why;
        VerbsProvider* p = default_provider(&why);
        if (p) return py::make_tuple(p->provider_name(), std::string());
        return py::make_tuple(py::none(), why);
    });
    m.def("rdma_devices", [] {
        VerbsProvider* p = default_provider(nullptr);
        return p ? p->list_devices() : std::vector<std::string>{};
    });
    m.def("rdma_loopback_inject_error", [](int op, int status, int count) { loopback_inject_error(static_cast<WrOp>(op), status, count); },
          py::arg("wr_op"), py::arg("status"), py::arg("count") = 1);
    m.def("rdma_loopback_stats", [] {
        py::dict d;
        d["executed_wrs"] = loopback_executed_wrs();
        d["rnr_events"]   = loopback_rnr_events();
        return d;
    });
    m.def("rdma_worker_stats", [](int numa) {
        auto     w = RdmaWorker::for_node(numa);
        py::dict d;
        d["loops"]  = w->loops();
        d["sleeps"] = w->sleeps();
        return d;
    }, py::arg("numa_node") = -1);
    // The transport is always compiled in; whether it can run is a property of the host (rdma_provider()).
    m.attr("_BUILD_RDMA") = py::bool_(true);
}
