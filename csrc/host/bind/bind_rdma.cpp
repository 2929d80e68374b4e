// Bindings of the RDMA transport: the endpoint, its context, and the provider controls.
#include "bind/bind_common.h"
#include "transport/rdma/rdma_endpoint.h"
#include "transport/rdma/rdma_worker.h"

using namespace slime;
using namespace slime::rdma;

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

    py::class_<RdmaEndpoint, Endpoint, std::shared_ptr<RdmaEndpoint>>(m, "RDMAEndpoint")
        .def(py::init([](const std::string& dev, int port, const std::string& link, int num_qp) {
                 return RdmaEndpoint::create(dev, port, link, num_qp);
             }),
             py::arg("device") = "", py::arg("ib_port") = 1, py::arg("link_type") = "", py::arg("num_qp") = 0)
        .def("num_qp", &RdmaEndpoint::num_qp)
        .def("context", &RdmaEndpoint::context)
        .def("process", &RdmaEndpoint::process)
        .def("cancel_all", &RdmaEndpoint::cancel_all, py::call_guard<py::gil_scoped_release>())
        .def("posted_wrs", &RdmaEndpoint::posted_wrs)
        .def("signaled_wrs", &RdmaEndpoint::signaled_wrs)
        .def("credit_stalls", &RdmaEndpoint::credit_stalls);

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
