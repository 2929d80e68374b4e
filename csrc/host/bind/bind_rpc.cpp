// Python surface of the SlimeRPC session (`_slime_c.rpc`). Payloads enter as any object with
// the buffer protocol and leave as one `bytes` built from the receive slot; the GIL is
// released around every blocking wait and re-taken only to run Python writers.
#include "bind/bind_common.h"
#include "rpc/rpc_session.h"

using namespace slime;
using namespace slime::rpc;

namespace {

py::bytes wait_bytes(ClientFuture& f)
{
    {
        py::gil_scoped_release nogil;
        f.wait_for(-1);
    }
    if (!f.error().empty()) throw std::runtime_error(f.error());
    return py::bytes(f.payload());
}

Writer python_writer(py::function fn)
{
    // The Python callable receives (address, capacity) and returns the bytes it wrote.
    std::shared_ptr<py::function> h(new py::function(std::move(fn)), [](py::function* f) {
        py::gil_scoped_acquire gil;
        delete f;
    });
    return [h](char* dst, size_t cap) -> size_t {
        py::gil_scoped_acquire gil;
        return (*h)(reinterpret_cast<uintptr_t>(dst), cap).cast<size_t>();
    };
}

}  // namespace

void bind_rpc(py::module_& m)
{
    py::module_ r            = m.def_submodule("rpc", "SlimeRPC C++ backend");
    r.attr("WIRE_VERSION")   = WIRE_VERSION;
    r.attr("HEADER_SIZE")    = HEADER_SIZE;
    r.attr("EXC_BIT")        = EXC_BIT;
    r.attr("ACK_BIT")        = ACK_BIT;
    r.attr("REPLY_BIT")      = REPLY_BIT;
    r.attr("CHUNK_BIT")      = CHUNK_BIT;
    r.attr("LAST_BIT")       = LAST_BIT;
    r.attr("FLAG_MASK")      = FLAG_MASK;
    r.attr("MAX_SLOT_COUNT") = MAX_SLOT_COUNT;

    py::class_<ClientFuture, std::shared_ptr<ClientFuture>>(r, "ClientFuture")
        .def("wait", &wait_bytes)
        .def(
            "wait_for",
            [](ClientFuture& f, double timeout_seconds) -> py::object {
                bool done;
                {
                    py::gil_scoped_release nogil;
                    done = f.wait_for(static_cast<int64_t>(std::max(0.0, timeout_seconds) * 1000.0));
                }
                if (!done) return py::none();
                if (!f.error().empty()) throw std::runtime_error(f.error());
                return py::bytes(f.payload());
            },
            py::arg("timeout_seconds"))
        .def("done", &ClientFuture::done)
        .def("has_exception", &ClientFuture::has_exception)
        .def("rethrow_if_failed", [](ClientFuture& f) { if (f.done() && !f.error().empty()) throw std::runtime_error(f.error()); })
        .def_property_readonly("is_remote_exception", &ClientFuture::is_remote_exception)
        .def_property_readonly("request_id", &ClientFuture::request_id)
        .def_property_readonly("slot_id", &ClientFuture::slot_id);

    py::class_<InboundRequest>(r, "InboundRequest")
        .def_readonly("raw_tag", &InboundRequest::raw_tag)
        .def_readonly("base_tag", &InboundRequest::base_tag)
        .def_readonly("request_id", &InboundRequest::request_id)
        .def_readonly("slot_id", &InboundRequest::slot_id)
        .def_property_readonly("payload_ptr", [](const InboundRequest& q) { return reinterpret_cast<uintptr_t>(q.payload_ptr); })
        .def_property_readonly("payload_nbytes", [](const InboundRequest& q) { return q.payload_nbytes; })
        .def_property_readonly("payload", [](const InboundRequest& q) { return py::bytes(q.payload_ptr, q.payload_nbytes); });

    py::class_<RpcSession, std::shared_ptr<RpcSession>>(r, "RpcSession")
        .def(py::init<std::shared_ptr<Endpoint>, int, uintptr_t, int, uintptr_t, int, size_t, size_t, bool>(), py::arg("endpoint"),
             py::arg("local_send_handler"), py::arg("local_send_ptr"), py::arg("local_recv_handler"), py::arg("local_recv_ptr"),
             py::arg("remote_recv_handler"), py::arg("slot_size"), py::arg("slot_count"), py::arg("start_recv_pump") = true)
        .def(
            "call",
            [](RpcSession& s, uint32_t tag, py::buffer payload) {
                py::buffer_info info = payload.request();
                const void*     p    = info.ptr;
                const size_t    n    = static_cast<size_t>(info.size) * static_cast<size_t>(info.itemsize);
                py::gil_scoped_release nogil;
                return s.call(tag, p, n);
            },
            py::arg("tag"), py::arg("payload"))
        .def(
            "call_inplace",
            [](RpcSession& s, uint32_t tag, py::function writer) {
                Writer w = python_writer(std::move(writer));
                py::gil_scoped_release nogil;
                return s.call_inplace(tag, w);
            },
            py::arg("tag"), py::arg("writer"))
        .def(
            "post_reply",
            [](RpcSession& s, uint32_t tag, uint64_t request_id, uint32_t slot, py::buffer payload) {
                py::buffer_info info = payload.request();
                const void*     p    = info.ptr;
                const size_t    n    = static_cast<size_t>(info.size) * static_cast<size_t>(info.itemsize);
                py::gil_scoped_release nogil;
                s.post_reply(tag, request_id, slot, p, n);
            },
            py::arg("tag"), py::arg("request_id"), py::arg("client_slot_id"), py::arg("payload"))
        .def(
            "post_reply_inplace",
            [](RpcSession& s, uint32_t tag, uint64_t request_id, uint32_t slot, py::function writer) {
                Writer w = python_writer(std::move(writer));
                py::gil_scoped_release nogil;
                s.post_reply_inplace(tag, request_id, slot, w);
            },
            py::arg("tag"), py::arg("request_id"), py::arg("client_slot_id"), py::arg("writer"))
        .def(
            "poll_request",
            [](RpcSession& s, double timeout) -> py::object {
                std::optional<InboundRequest> q;
                {
                    py::gil_scoped_release nogil;
                    q = s.poll_request(timeout < 0 ? -1 : static_cast<int64_t>(timeout * 1000));
                }
                if (!q) return py::none();
                return py::cast(*q);
            },
            py::arg("timeout") = -1.0)
        .def("close", &RpcSession::close, py::call_guard<py::gil_scoped_release>())
        .def("detach_request", &RpcSession::detach_request, py::arg("request_id"))
        .def_property_readonly("slot_count", &RpcSession::slot_count)
        .def_property_readonly("slot_size", &RpcSession::slot_size)
        .def_property_readonly("payload_capacity", &RpcSession::payload_capacity)
        .def_property_readonly("closed", &RpcSession::closed)
        .def_property_readonly("requests_sent", &RpcSession::requests_sent)
        .def_property_readonly("replies_received", &RpcSession::replies_received)
        .def_property_readonly("requests_received", &RpcSession::requests_received);
}
