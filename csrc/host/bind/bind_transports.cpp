// Bindings of the optional transports: the Ascend Direct stub (interface only) and the RDMA
// RC endpoint, which is present when libibverbs can be loaded at run time.
#include "bind/bind_common.h"
#include "transport/ascend_stub.h"

using namespace slime;

void bind_rdma(py::module_& m);

void bind_extra_transports(py::module_& m)
{
    py::class_<AscendDirectEndpoint, std::shared_ptr<AscendDirectEndpoint>>(m, "AscendDirectEndpoint")
        .def(py::init<>())
        .def("init", &AscendDirectEndpoint::init, py::arg("host"), py::arg("port"))
        .def("register_memory_region", &AscendDirectEndpoint::register_memory_region, py::arg("addr"), py::arg("offset"),
             py::arg("length"), py::arg("name") = std::nullopt)
        .def("get_mr_handle", &AscendDirectEndpoint::get_mr_handle)
        .def("endpoint_info", &AscendDirectEndpoint::endpoint_info)
        .def("mr_info", &AscendDirectEndpoint::mr_info)
        .def("connect", [](AscendDirectEndpoint& e, const Json& info) { return e.connect(info); })
        .def("read", [](AscendDirectEndpoint& e, py::object, py::object) { e.read(); }, py::arg("assign"), py::arg("stream") = py::none());
    m.attr("_BUILD_ASCEND_DIRECT") = false;
#ifndef SLIME_NO_RDMA
    bind_rdma(m);
#else
    // built with BUILD_RDMA=OFF: the probes answer, the classes are absent
    m.attr("_BUILD_RDMA") = py::bool_(false);
    m.def("rdma_devices", [] { return std::vector<std::string>{}; });
    m.def("rdma_provider", []() -> py::tuple { return py::make_tuple(py::none(), std::string("built without the RDMA transport (BUILD_RDMA=OFF)")); });
#endif
}
