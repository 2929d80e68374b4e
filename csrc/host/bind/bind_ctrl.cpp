// Python surface of the control plane (`_slime_c.ctrl`): the embedded NanoCtrl server and
// its key-value store (used directly by in-process PeerAgents and by tests with a fake clock).
#include "bind/bind_common.h"
#include "ctrl/kvstore.h"
#include "ctrl/nanoctrl.h"
#include "ctrl/net_server.h"
#include "ctrl/obs_view.h"

using namespace slime;
using namespace slime::ctrl;

namespace {

py::object opt_str(const std::optional<std::string>& v)
{
    if (!v) return py::none();
    return py::str(*v);
}

py::list entries_to_py(const std::vector<StreamEntry>& es)
{
    py::list out;
    for (const auto& e : es) {
        py::dict f;
        for (const auto& kv : e.fields) f[py::str(kv.first)] = py::str(kv.second);
        out.append(py::make_tuple(e.id.str(), f));
    }
    return out;
}

// Python callables kept by C++ threads: copies of the holder never touch the reference count, and the
// last owner drops the callable with the GIL held.
std::shared_ptr<py::function> hold(py::function fn)
{
    return std::shared_ptr<py::function>(new py::function(std::move(fn)), [](py::function* f) {
        py::gil_scoped_acquire gil;
        delete f;
    });
}

std::vector<std::pair<std::string, std::string>> dict_fields(const py::dict& d)
{
    std::vector<std::pair<std::string, std::string>> f;
    for (auto item : d) f.emplace_back(py::str(item.first).cast<std::string>(), py::str(item.second).cast<std::string>());
    return f;
}

}  // namespace

void bind_ctrl(py::module_& m)
{
    py::module_ c = m.def_submodule("ctrl", "Embedded control plane: NanoCtrl + Redis-semantics store");
    c.attr("ENTITY_TTL_SECS") = kEntityTtlSecs;

    py::class_<KvStore, std::shared_ptr<KvStore>>(c, "KvStore")
        .def(py::init<>())
        .def("set_clock", [](KvStore& s, py::function fn) {
            auto h = hold(std::move(fn));
            s.set_clock([h]() -> int64_t {
                py::gil_scoped_acquire gil;
                return (*h)().cast<int64_t>();
            });
        })
        .def("now_ms", &KvStore::now_ms)
        .def("set", &KvStore::set, py::arg("key"), py::arg("value"), py::arg("px") = -1, py::arg("nx") = false, py::call_guard<py::gil_scoped_release>())
        .def("get", [](KvStore& s, const std::string& k) { return opt_str(s.get(k)); })
        .def("mget", [](KvStore& s, const std::vector<std::string>& ks) {
            py::list out;
            for (auto& v : s.mget(ks)) out.append(opt_str(v));
            return out;
        })
        .def("delete", [](KvStore& s, py::args keys) {
            std::vector<std::string> ks;
            for (auto k : keys) ks.push_back(py::str(k).cast<std::string>());
            return s.del(ks);
        })
        .def("exists", &KvStore::exists, py::call_guard<py::gil_scoped_release>())
        .def("pexpire", &KvStore::expire, py::call_guard<py::gil_scoped_release>())
        .def("expire", [](KvStore& s, const std::string& k, int64_t secs) { return s.expire(k, secs * 1000); }, py::call_guard<py::gil_scoped_release>())
        .def("pttl", &KvStore::pttl, py::call_guard<py::gil_scoped_release>())
        .def("incr", &KvStore::incr, py::arg("key"), py::arg("by") = 1, py::call_guard<py::gil_scoped_release>())
        .def("keys", &KvStore::keys, py::arg("pattern") = "*", py::call_guard<py::gil_scoped_release>())
        .def("scan", &KvStore::scan, py::arg("cursor") = 0, py::arg("match") = "*", py::arg("count") = 10, py::call_guard<py::gil_scoped_release>())
        .def("type", &KvStore::type_of)
        .def("flushall", &KvStore::flush_all)
        .def("dbsize", &KvStore::size)
        .def("hset", [](KvStore& s, const std::string& k, const py::dict& mapping) { return s.hset(k, dict_fields(mapping)); },
             py::arg("key"), py::arg("mapping"))
        .def("hget", [](KvStore& s, const std::string& k, const std::string& f) { return opt_str(s.hget(k, f)); })
        .def("hgetall", [](KvStore& s, const std::string& k) {
            py::dict d;
            for (auto& kv : s.hgetall(k)) d[py::str(kv.first)] = py::str(kv.second);
            return d;
        })
        .def("hdel", [](KvStore& s, const std::string& k, py::args fields) {
            std::vector<std::string> fs;
            for (auto f : fields) fs.push_back(py::str(f).cast<std::string>());
            return s.hdel(k, fs);
        })
        .def("lpush", [](KvStore& s, const std::string& k, py::args vs) {
            std::vector<std::string> v;
            for (auto x : vs) v.push_back(py::str(x).cast<std::string>());
            return s.lpush(k, v);
        })
        .def("rpush", [](KvStore& s, const std::string& k, py::args vs) {
            std::vector<std::string> v;
            for (auto x : vs) v.push_back(py::str(x).cast<std::string>());
            return s.rpush(k, v);
        })
        .def("lpop", [](KvStore& s, const std::string& k) { return opt_str(s.lpop(k)); })
        .def("rpop", [](KvStore& s, const std::string& k) { return opt_str(s.rpop(k)); })
        .def("llen", &KvStore::llen)
        .def("lrange", &KvStore::lrange)
        .def(
            "blpop",
            [](KvStore& s, const std::vector<std::string>& keys, double timeout) -> py::object {
                std::optional<std::pair<std::string, std::string>> r;
                {
                    py::gil_scoped_release nogil;
                    r = s.blpop(keys, static_cast<int64_t>(timeout * 1000));
                }
                if (!r) return py::none();
                return py::make_tuple(r->first, r->second);
            },
            py::arg("keys"), py::arg("timeout") = 0.0)
        .def("xadd", [](KvStore& s, const std::string& k, const py::dict& fields, const std::string& id, size_t maxlen) {
            const std::string got = s.xadd(k, id, dict_fields(fields), maxlen);
            if (got.empty()) throw std::runtime_error("ERR The ID specified in XADD is equal or smaller than the target stream top item");
            return got;
        }, py::arg("key"), py::arg("fields"), py::arg("id") = "*", py::arg("maxlen") = 0)
        .def("xlen", &KvStore::xlen)
        .def(
            "xread",
            [](KvStore& s, const py::dict& streams, size_t count, py::object block) {
                std::vector<std::pair<std::string, std::string>> ki;
                for (auto item : streams) ki.emplace_back(py::str(item.first).cast<std::string>(), py::str(item.second).cast<std::string>());
                const int64_t block_ms = block.is_none() ? -1 : block.cast<int64_t>();
                std::vector<std::pair<std::string, std::vector<StreamEntry>>> res;
                {
                    py::gil_scoped_release nogil;
                    res = s.xread(ki, count, block_ms);
                }
                py::list out;
                for (auto& r : res) out.append(py::make_tuple(r.first, entries_to_py(r.second)));
                return out;
            },
            py::arg("streams"), py::arg("count") = 0, py::arg("block") = py::none())
        .def("xrange", [](KvStore& s, const std::string& k, const std::string& a, const std::string& b, size_t count) {
            return entries_to_py(s.xrange(k, a, b, count));
        }, py::arg("key"), py::arg("min") = "-", py::arg("max") = "+", py::arg("count") = 0)
        .def("publish", &KvStore::publish)
        .def("subscribe", [](KvStore& s, const std::string& channel, py::function fn) {
            auto h = hold(std::move(fn));
            return s.subscribe(channel, [h](const std::string& ch, const std::string& msg) {
                py::gil_scoped_acquire gil;
                (*h)(ch, msg);
            });
        })
        .def("unsubscribe", &KvStore::unsubscribe)
        .def("interrupt", &KvStore::interrupt)
        .def_static("glob_match", &KvStore::glob_match);

    py::class_<NanoCtrl, std::shared_ptr<NanoCtrl>>(c, "NanoCtrl")
        .def(py::init<>())
        .def("start", &NanoCtrl::start, py::arg("host") = "127.0.0.1", py::arg("http_port") = 0, py::arg("resp_port") = 0,
             py::arg("public_host") = "", py::call_guard<py::gil_scoped_release>())
        .def("stop", &NanoCtrl::stop, py::call_guard<py::gil_scoped_release>())
        .def("running", &NanoCtrl::running)
        .def_property_readonly("http_port", &NanoCtrl::http_port)
        .def_property_readonly("resp_port", &NanoCtrl::resp_port)
        .def_property_readonly("store", &NanoCtrl::store)
        .def(
            "handle",
            [](NanoCtrl& n, const std::string& method, const std::string& path, const std::string& body) {
                HttpRequest q;
                q.method = method;
                q.path   = path;
                q.body   = body;
                HttpResponse r;
                {
                    py::gil_scoped_release nogil;
                    r = n.handle(q);
                }
                return py::make_tuple(r.status, r.body);
            },
            py::arg("method"), py::arg("path"), py::arg("body") = "", "Dispatch one request without going through a socket.");

    c.def("snapshot_state", &snapshot_state, py::arg("snapshot"), py::arg("now_ms"), py::arg("stale_ms") = 45000);
    c.def("human_bps", &human_bps);
    c.def("human_bytes", &human_bytes);
    c.def("obs_view", [](const std::string& address, const std::string& scope, const std::string& view, int64_t stale_ms, bool as_json) {
        std::vector<PeerSnapshot> peers;
        {
            py::gil_scoped_release nogil;
            peers = fetch_snapshots(address, scope, stale_ms);
        }
        return render_obs_view(peers, view, as_json);
    }, py::arg("address"), py::arg("scope") = "", py::arg("view") = "status", py::arg("stale_ms") = 45000, py::arg("as_json") = false);

    py::class_<RespServer, std::shared_ptr<RespServer>>(c, "RespServer")
        .def(py::init<std::shared_ptr<KvStore>>())
        .def("start", &RespServer::start, py::arg("host") = "127.0.0.1", py::arg("port") = 0)
        .def("stop", &RespServer::stop, py::call_guard<py::gil_scoped_release>())
        .def_property_readonly("port", &RespServer::port)
        .def("execute", [](RespServer& s, const std::vector<std::string>& argv) {
            std::string out;
            {
                py::gil_scoped_release nogil;
                out = s.execute(argv);
            }
            return py::bytes(out);
        });
}
