// The C function table of csrc/include/slime_bridge.h over the endpoints of this library, and its Python accessor.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>

#include "bind_common.h"
#include "slime_bridge.h"
#include "transport/endpoint.h"
#ifndef SLIME_NO_RDMA
#include "transport/rdma/rdma_endpoint.h"
#include "transport/rdma/verbs.h"
#endif
#include "transport/tcp_endpoint.h"

namespace slime {
#ifndef SLIME_NO_RDMA
using namespace slime::rdma;
#endif
namespace {

struct EpBox {
    std::shared_ptr<Endpoint> ep;
    std::string               kind;
};
struct FutBox {
    std::shared_ptr<OpFuture> fut;
};

void set_err(char* err, size_t n, const std::string& msg)
{
    if (err && n) std::snprintf(err, n, "%s", msg.c_str());
}

void* b_endpoint_create(const char* transport, const char* bind_host, int rank, char* err, size_t err_len)
{
    try {
        const std::string want = transport ? transport : "";
        std::vector<std::string> devices;
        std::string              provider_name;
#ifndef SLIME_NO_RDMA
        if (want != "tcp") {
            if (VerbsProvider* p = default_provider(nullptr)) {
                devices       = p->list_devices();
                provider_name = p->provider_name();
            }
        }
#endif
        if (want == "rdma" && devices.empty()) {
            set_err(err, err_len, "transport rdma was asked for but no verbs provider with a device exists");
            return nullptr;
        }
        auto box = std::make_unique<EpBox>();
#ifndef SLIME_NO_RDMA
        if (!devices.empty() && (want == "rdma" || provider_name == "ibverbs"))
            box->ep = RdmaEndpoint::create(devices[static_cast<size_t>(rank < 0 ? 0 : rank) % devices.size()], 1, "", 0);
        else
#endif
            box->ep = std::make_shared<TcpEndpoint>(bind_host && *bind_host ? bind_host : "127.0.0.1", 0, 1);
        box->kind = box->ep->kind();
        return box.release();
    }
    catch (const std::exception& e) {
        set_err(err, err_len, e.what());
        return nullptr;
    }
}

void b_endpoint_destroy(void* h)
{
    auto* box = static_cast<EpBox*>(h);
    if (!box) return;
    try {
        box->ep->shutdown();
    }
    catch (...) {
    }
    delete box;
}

char* b_endpoint_info(void* h)
{
    const std::string s = static_cast<EpBox*>(h)->ep->endpoint_info().dump();
    char*             out = static_cast<char*>(std::malloc(s.size() + 1));
    if (out) std::memcpy(out, s.c_str(), s.size() + 1);
    return out;
}

int b_endpoint_connect(void* h, const char* info_json, char* err, size_t err_len)
{
    try {
        const int rc = static_cast<EpBox*>(h)->ep->connect(Json::parse(info_json));
        if (rc != 0) set_err(err, err_len, "the endpoint refused the peer's description (wrong kind of endpoint, or unreachable); see the log");
        return rc;
    }
    catch (const std::exception& e) {
        set_err(err, err_len, e.what());
        return -1;
    }
}

const char* b_endpoint_kind(void* h)
{
    return static_cast<EpBox*>(h)->kind.c_str();
}

void* b_send(void* h, uintptr_t ptr, size_t length)
{
    try {
        return new FutBox{static_cast<EpBox*>(h)->ep->send(chunk_tuple_t{ptr, 0, length}, nullptr)};
    }
    catch (...) {
        return nullptr;
    }
}

void* b_recv(void* h, uintptr_t ptr, size_t length)
{
    try {
        return new FutBox{static_cast<EpBox*>(h)->ep->recv(chunk_tuple_t{ptr, 0, length}, nullptr)};
    }
    catch (...) {
        return nullptr;
    }
}

int b_future_wait(void* f, int64_t timeout_ms)
{
    try {
        return static_cast<FutBox*>(f)->fut->wait(timeout_ms);
    }
    catch (...) {
        return FAILED;
    }
}

int b_future_done(void* f)
{
    return static_cast<FutBox*>(f)->fut->done() ? 1 : 0;
}

void b_future_free(void* f)
{
    delete static_cast<FutBox*>(f);
}

void b_free_string(char* s)
{
    std::free(s);
}

}  // namespace

extern const SlimeBridge kBridgeTable = {SLIME_BRIDGE_VERSION, b_endpoint_create, b_endpoint_destroy, b_endpoint_info, b_endpoint_connect,
                             b_endpoint_kind,      b_send,            b_recv,             b_future_wait,   b_future_done,
                             b_future_free,        b_free_string};

}  // namespace slime

void bind_bridge(py::module_& m)
{
    m.def("bridge_table", [] { return reinterpret_cast<uintptr_t>(&slime::kBridgeTable); },
          "Address of the C function table over this module's endpoints (csrc/include/slime_bridge.h)");
}
