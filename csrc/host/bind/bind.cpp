// Python module `_slime_c`: the host runtime. Names follow the reference's module of the
// same name (dlslime/csrc/python/bind.cpp:98-557 in the reference) where a counterpart
// exists: OpCode, Assignment, cache.*, rpc.*, discover_topology, obs_*, the future
// classes. Blocking calls release the GIL.
#include "bind/bind_common.h"

#include "cache/cache_server.h"
#include "core/env.h"
#include "engine/assignment.h"
#include "engine/future.h"
#include "engine/memory_pool.h"
#include "obs/obs.h"
#include "topology/topology.h"
#include "transport/endpoint.h"
#include "transport/tcp_endpoint.h"

using namespace slime;

void bind_rpc(py::module_& m);
void bind_ctrl(py::module_& m);
void bind_extra_transports(py::module_& m);
void bind_bridge(py::module_& m);

static void bind_cache(py::module_& m)
{
    using namespace slime::cache;
    py::module_ sub = m.def_submodule("cache", "DLSlimeCache directory primitives.");
    py::class_<AssignmentManifest>(sub, "AssignmentManifest")
        .def(py::init<>())
        .def_readwrite("peer_agent_id", &AssignmentManifest::peer_agent_id)
        .def_readwrite("assignments", &AssignmentManifest::assignments)
        .def_readwrite("slab_ids", &AssignmentManifest::slab_ids)
        .def_readwrite("version", &AssignmentManifest::version)
        .def("total_bytes", &AssignmentManifest::total_bytes)
        .def("__repr__", [](const AssignmentManifest& x) {
            return "AssignmentManifest(peer_agent_id='" + x.peer_agent_id + "', version=" + std::to_string(x.version)
                   + ", #assignments=" + std::to_string(x.assignments.size()) + ", total_bytes=" + std::to_string(x.total_bytes()) + ")";
        });
    py::class_<CacheStats>(sub, "CacheStats")
        .def_readonly("num_assignment_peers", &CacheStats::num_assignment_peers)
        .def_readonly("num_assignment_entries", &CacheStats::num_assignment_entries)
        .def_readonly("num_assignments", &CacheStats::num_assignments)
        .def_readonly("assignment_bytes", &CacheStats::assignment_bytes)
        .def_readonly("slab_size", &CacheStats::slab_size)
        .def_readonly("memory_size", &CacheStats::memory_size)
        .def_readonly("num_slabs", &CacheStats::num_slabs)
        .def_readonly("used_slabs", &CacheStats::used_slabs)
        .def_readonly("free_slabs", &CacheStats::free_slabs);
    py::class_<CacheServer>(sub, "CacheServer")
        .def(py::init<uint64_t, uint64_t>(), py::arg("slab_size") = CacheServer::kDefaultSlabSize,
             py::arg("memory_size") = CacheServer::kDefaultMemorySize)
        .def("slab_size", &CacheServer::slab_size)
        .def("memory_size", &CacheServer::memory_size)
        .def("num_slabs", &CacheServer::num_slabs)
        .def("store_assignments", &CacheServer::store_assignments, py::arg("peer_agent_id"), py::arg("assignments"))
        .def("query_assignments", &CacheServer::query_assignments, py::arg("peer_agent_id"), py::arg("version"))
        .def("delete_assignments", &CacheServer::erase_assignments, py::arg("peer_agent_id"), py::arg("version"))
        .def("stats", &CacheServer::stats)
        .def("clear", &CacheServer::clear);
}

template<typename Fut>
static void bind_future(py::module_& m, const char* name)
{
    py::class_<Fut, std::shared_ptr<Fut>>(m, name)
        .def("wait", [](const Fut& f, double timeout) { return f.wait(timeout < 0 ? -1 : static_cast<int64_t>(timeout * 1000)); },
             py::arg("timeout") = -1.0, py::call_guard<py::gil_scoped_release>(),
             "Block until the operation completed; returns the status (0 ok, 402 timeout, 403 failed).")
        .def("done", &Fut::done)
        .def("wait_on_stream", &Fut::wait_on_stream, py::arg("limit_ms") = 0.0,
             "Make the stream given at submission wait on the device for this operation (stream-ordered signals only). "
             "The wait is bounded (limit_ms, else SLIME_STREAM_WAIT_MS, else 1 s); if it runs out, wait() returns 402.")
        .def("stream_wait_timed_out", &Fut::stream_wait_timed_out);
}

PYBIND11_MODULE(_slime_c, m)
{
    m.doc() = "Host runtime of the B200-native DLSlime-capability framework";
    m.attr("_BUILD_NVLINK")    = true;   // the NVLink endpoint lives in libslime_cuda (dlslime_b200.ops.nvlink)
    m.attr("_BUILD_TCP")       = true;
    m.attr("_BUILD_INTRA_OPS") = true;   // dlslime_b200.ops: all-gather, EP dispatch/combine, AG-GEMM
    m.attr("_BUILD_INTER_OPS") = false;
    m.attr("_BUILD_RPC")       = true;
    m.attr("_BUILD_NVTX")      = slime::kNvtxCompiledIn;  // NVTX ranges around the signal operations (core/nvtx.h)

    m.def(
        "discover_topology",
        [](std::optional<std::string> preferred_device, int ib_port, std::optional<std::string> preferred_link_type,
           const std::string& sysfs_root, std::optional<std::vector<std::string>> devices, const std::string& procfs_root,
           bool allow_software_links) {
            topology::Options o;
            o.preferred_device     = std::move(preferred_device);
            o.ib_port              = ib_port;
            o.preferred_link_type  = std::move(preferred_link_type);
            o.sysfs_root           = sysfs_root;
            o.procfs_root          = procfs_root;
            o.devices              = std::move(devices);
            o.allow_software_links = allow_software_links;
            return topology::discover(o);
        },
        py::arg("preferred_device") = std::nullopt, py::arg("ib_port") = 1, py::arg("preferred_link_type") = std::nullopt,
        py::arg("sysfs_root") = "/sys", py::arg("devices") = std::nullopt, py::arg("procfs_root") = "/proc",
        py::arg("allow_software_links") = false);
    m.def("available_nic", [] { return topology::list_rdma_devices("/sys"); });
    m.def("socket_id", [](const std::string& dev) { return topology::numa_node_of(dev, "/sys"); });

    py::enum_<OpCode>(m, "OpCode")
        .value("READ", OpCode::READ)
        .value("WRITE", OpCode::WRITE)
        .value("WRITE_WITH_IMM_DATA", OpCode::WRITE_WITH_IMM)
        .value("SEND", OpCode::SEND)
        .value("RECV", OpCode::RECV);

    py::class_<Assignment>(m, "Assignment")
        .def(py::init<uintptr_t, uint64_t, uint64_t, uint64_t>())
        .def(py::init<uintptr_t, uintptr_t, uint64_t, uint64_t, uint64_t>())
        .def_readwrite("mr_key", &Assignment::mr_key)
        .def_readwrite("remote_mr_key", &Assignment::remote_mr_key)
        .def_readwrite("target_offset", &Assignment::target_offset)
        .def_readwrite("source_offset", &Assignment::source_offset)
        .def_readwrite("length", &Assignment::length)
        .def("dump", &Assignment::dump)
        .def("to_tuple", [](const Assignment& a) { return py::make_tuple(a.mr_key, a.remote_mr_key, a.target_offset, a.source_offset, a.length); })
        .def("__repr__", [](const Assignment& a) { return "Assignment(" + a.dump() + ")"; });
    m.def("split_assign_by_max_length", [](const AssignmentBatch& b, size_t max_length) {
        AssignmentBatch out;
        split_assign_by_max_length(b, out, max_length);
        return out;
    });
    m.def("split_assign_by_step", [](const AssignmentBatch& b, size_t step) {
        std::vector<AssignmentBatch> out;
        split_assign_by_step(b, out, step);
        return out;
    });
    m.def("nsplit_assign_by_step", [](const AssignmentBatch& b, size_t nstep) {
        std::vector<AssignmentBatch> out;
        nsplit_assign_by_step(b, out, nstep);
        return out;
    });

    bind_cache(m);

    py::class_<DeviceSignal, std::shared_ptr<DeviceSignal>>(m, "DeviceSignal")
        .def("wait", [](DeviceSignal& s, uint32_t mask, double timeout) { return s.wait_comm_done_cpu(mask, timeout < 0 ? -1 : static_cast<int64_t>(timeout * 1000)); },
             py::arg("mask") = 1, py::arg("timeout") = -1.0, py::call_guard<py::gil_scoped_release>())
        .def("set_comm_done", &DeviceSignal::set_comm_done)
        .def("record_gpu_ready", &DeviceSignal::record_gpu_ready)
        .def("is_gpu_ready", &DeviceSignal::is_gpu_ready)
        .def("get_comm_done_mask", &DeviceSignal::get_comm_done_mask)
        .def("force_complete", &DeviceSignal::force_complete)
        .def("bind_stream", [](DeviceSignal& s, uintptr_t stream) { s.bind_stream(reinterpret_cast<void*>(stream)); })
        .def("wait_comm_done_on_stream", &DeviceSignal::wait_comm_done_on_stream, py::arg("mask") = 1)
        .def("stream_wait_timed_out", &DeviceSignal::stream_wait_timed_out)
        .def("set_stream_wait_limit_ms", [](DeviceSignal& s, double ms) { s.set_stream_wait_limit_ns(static_cast<unsigned long long>(ms * 1e6)); })
        .def("reset_all", &DeviceSignal::reset_all);
    // Addresses of four C functions (see StreamHooks); the kernel library's loader passes its own.
    m.def("install_stream_hooks", [](uintptr_t alloc_words, uintptr_t free_words, uintptr_t record_value, uintptr_t wait_mask) {
        StreamHooks& h = stream_hooks();
        h.alloc_words  = reinterpret_cast<decltype(h.alloc_words)>(alloc_words);
        h.free_words   = reinterpret_cast<decltype(h.free_words)>(free_words);
        h.record_value = reinterpret_cast<decltype(h.record_value)>(record_value);
        h.wait_mask    = reinterpret_cast<decltype(h.wait_mask)>(wait_mask);
    });
    m.def("stream_hooks_installed", [] { return stream_hooks().installed(); });
    m.def("create_signal", [](bool bypass) { return create_signal(bypass); }, py::arg("bypass") = true);

    bind_future<OpFuture>(m, "SlimeSendFuture");
    m.attr("SlimeRecvFuture") = m.attr("SlimeSendFuture");
    py::class_<ReadWriteFuture, std::shared_ptr<ReadWriteFuture>>(m, "SlimeReadWriteFuture")
        .def("wait", [](const ReadWriteFuture& f, double timeout) { return f.wait(timeout < 0 ? -1 : static_cast<int64_t>(timeout * 1000)); },
             py::arg("timeout") = -1.0, py::call_guard<py::gil_scoped_release>())
        .def("done", &ReadWriteFuture::done)
        .def("wait_on_stream", &ReadWriteFuture::wait_on_stream, py::arg("limit_ms") = 0.0)
        .def("stream_wait_timed_out", &ReadWriteFuture::stream_wait_timed_out);
    py::class_<ImmRecvFuture, std::shared_ptr<ImmRecvFuture>>(m, "SlimeImmRecvFuture")
        .def("wait", [](const ImmRecvFuture& f, double timeout) { return f.wait(timeout < 0 ? -1 : static_cast<int64_t>(timeout * 1000)); },
             py::arg("timeout") = -1.0, py::call_guard<py::gil_scoped_release>())
        .def("done", &ImmRecvFuture::done)
        .def("wait_on_stream", &ImmRecvFuture::wait_on_stream, py::arg("limit_ms") = 0.0)
        .def("stream_wait_timed_out", &ImmRecvFuture::stream_wait_timed_out)
        .def("imm_data", &ImmRecvFuture::imm_data)
        .def("time_trace_enabled", &ImmRecvFuture::time_trace_enabled)
        .def("time_trace_start_ns", &ImmRecvFuture::time_trace_start_ns)
        .def("time_trace_end_ns", &ImmRecvFuture::time_trace_end_ns)
        .def("time_trace_elapsed_ns", &ImmRecvFuture::time_trace_elapsed_ns);

    py::class_<LocalMemoryPool, std::shared_ptr<LocalMemoryPool>>(m, "MemoryPool")
        .def(py::init<>())
        .def("register_memory_region",
             [](LocalMemoryPool& p, uintptr_t ptr, uint64_t length, std::optional<std::string> name) { return p.register_memory_region(ptr, length, name); },
             py::arg("data_ptr"), py::arg("length"), py::arg("name") = std::nullopt)
        .def("get_handle", [](LocalMemoryPool& p, const std::string& name) { return p.get_mr_handle(name); })
        .def("unregister_memory_region",
             [](LocalMemoryPool& p, py::object key) {
                 if (py::isinstance<py::str>(key)) return p.unregister_memory_region(key.cast<std::string>());
                 return p.unregister_memory_region(key.cast<int32_t>());
             },
             py::arg("key"))
        .def("mr_info", &LocalMemoryPool::mr_info)
        .def("live_count", &LocalMemoryPool::live_count);

    using AssignVec = std::vector<assign_tuple_t>;
    py::class_<Endpoint, std::shared_ptr<Endpoint>>(m, "Endpoint")
        .def("kind", &Endpoint::kind)
        .def("connect", &Endpoint::connect, py::call_guard<py::gil_scoped_release>())
        .def("connected", &Endpoint::connected)
        .def("endpoint_info", &Endpoint::endpoint_info)
        .def("mr_info", &Endpoint::mr_info)
        .def("get_pool", &Endpoint::local_pool)
        .def("set_pool", &Endpoint::set_local_pool, py::arg("pool"))
        .def("register_memory_region",
             py::overload_cast<const std::string&, uintptr_t, uintptr_t, size_t>(&Endpoint::register_memory_region),
             py::arg("name"), py::arg("data_ptr"), py::arg("offset"), py::arg("length"))
        .def("register_memory_region", py::overload_cast<uintptr_t, uintptr_t, size_t>(&Endpoint::register_memory_region),
             py::arg("data_ptr"), py::arg("offset"), py::arg("length"))
        .def("unregister_memory_region",
             [](Endpoint& e, py::object key) {
                 if (py::isinstance<py::str>(key)) return e.local_pool()->unregister_memory_region(key.cast<std::string>());
                 return e.local_pool()->unregister_memory_region(key.cast<int32_t>());
             })
        .def("get_mr_handle", [](Endpoint& e, const std::string& n) { return e.local_pool()->get_mr_handle(n); })
        .def("get_remote_mr_handle", [](Endpoint& e, const std::string& n) { return e.remote_pool()->get_remote_mr_handle(n); })
        .def("register_remote_memory_region", &Endpoint::register_remote_memory_region, py::arg("name"), py::arg("mr_info"))
        .def("remote_mr_info", [](Endpoint& e) { return e.remote_pool()->remote_mr_info(); })
        .def("send", [](Endpoint& e, const chunk_tuple_t& c, uintptr_t stream) { return e.send(c, reinterpret_cast<void*>(stream)); },
             py::arg("chunk"), py::arg("stream_handler") = 0, py::call_guard<py::gil_scoped_release>())
        .def("recv", [](Endpoint& e, const chunk_tuple_t& c, uintptr_t stream) { return e.recv(c, reinterpret_cast<void*>(stream)); },
             py::arg("chunk"), py::arg("stream_handler") = 0, py::call_guard<py::gil_scoped_release>())
        .def("read", [](Endpoint& e, const AssignVec& a, uintptr_t stream) { return e.read(a, reinterpret_cast<void*>(stream)); },
             py::arg("assign"), py::arg("stream") = 0, py::call_guard<py::gil_scoped_release>())
        .def("write", [](Endpoint& e, const AssignVec& a, uintptr_t stream) { return e.write(a, reinterpret_cast<void*>(stream)); },
             py::arg("assign"), py::arg("stream") = 0, py::call_guard<py::gil_scoped_release>())
        .def("write_with_imm",
             [](Endpoint& e, const AssignVec& a, int32_t imm, uintptr_t stream) { return e.write_with_imm(a, imm, reinterpret_cast<void*>(stream)); },
             py::arg("assign"), py::arg("imm_data") = 0, py::arg("stream") = 0, py::call_guard<py::gil_scoped_release>())
        .def("imm_recv", [](Endpoint& e, uintptr_t stream) { return e.imm_recv(reinterpret_cast<void*>(stream)); },
             py::arg("stream") = 0, py::call_guard<py::gil_scoped_release>())
        .def("process", &Endpoint::process, py::call_guard<py::gil_scoped_release>())
        .def("cancel_all", &Endpoint::cancel_all, py::call_guard<py::gil_scoped_release>())
        .def("shutdown", &Endpoint::shutdown, py::call_guard<py::gil_scoped_release>());

    py::class_<TcpEndpoint, Endpoint, std::shared_ptr<TcpEndpoint>>(m, "TcpEndpoint")
        .def(py::init<const std::string&, int, int>(), py::arg("host") = "127.0.0.1", py::arg("port") = 0, py::arg("num_qp") = 1)
        .def("port", &TcpEndpoint::port)
        .def("host", &TcpEndpoint::host)
        .def("inject_fault", &TcpEndpoint::inject_fault, py::arg("what"), py::arg("count") = 1);

    // observability
    m.def("obs_enabled", &obs::enabled);
    m.def("obs_snapshot", &obs::snapshot);
    m.def("obs_reset_for_test", &obs::reset_for_test);
    m.def("obs_set_enabled_for_test", &obs::set_enabled_for_test);
    m.def("obs_register_nic_for_test", [](const std::string& name) { return obs::register_link(name, "rdma"); });
    m.def("obs_register_link", &obs::register_link, py::arg("name"), py::arg("kind") = "rdma");
    m.def("obs_record_submit", [](int link, int op, uint64_t n, uint64_t bytes) { obs::record_submit(link, static_cast<obs::OpIndex>(op), n, bytes); });
    m.def("obs_record_complete", [](int link, int op, uint64_t bytes) { obs::record_complete(link, static_cast<obs::OpIndex>(op), bytes); });
    m.def("obs_record_fail", [](int link, int op, uint64_t bytes) { obs::record_fail(link, static_cast<obs::OpIndex>(op), bytes); });

    m.def("engine_env", [] {
        const EngineEnv& e = engine_env();
        py::dict         d;
        d["SLIME_LOG_LEVEL"]                 = e.log_level;
        d["SLIME_MAX_LENGTH_PER_ASSIGNMENT"] = e.max_length_per_assignment;
        d["SLIME_MAX_SEND_WR"]               = e.max_send_wr;
        d["SLIME_QP_NUM"]                    = e.qp_num;
        d["SLIME_MAX_MSG_FIFO_DEPTH"]        = e.max_msg_fifo_depth;
        d["SLIME_MAX_IO_FIFO_DEPTH"]         = e.max_io_fifo_depth;
        d["SLIME_WITH_TIME_TRACE"]           = e.with_time_trace;
        d["SLIME_BYPASS_DEVICE_SIGNAL"]      = e.bypass_device_signal;
        return d;
    });

    bind_rpc(m);
    bind_ctrl(m);
    bind_extra_transports(m);
    bind_bridge(m);
}
