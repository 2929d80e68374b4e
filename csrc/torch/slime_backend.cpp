// torch.distributed backend "dlslime" in C++: a c10d::Backend whose send / recv run over this runtime's endpoints.
//
// Same contract as the reference's backend (dlslime/csrc/torch/slime_backend.{h,cpp} in the reference): one endpoint
// per peer built at construction, endpoint descriptions exchanged through the c10d store under
// SLIME_ENDPOINT_<rank>_<peer>, full mesh connected before the constructor returns, send / recv (and coalescing of
// them) only; every collective keeps c10d::Backend's "does not support" error. Differences, on purpose: every tensor of
// the list is transferred (the reference moves tensors[0] only), wait(timeout) honours its timeout (status 402 becomes
// an error), and the work returned by recv is tagged as a receive.
//
// This file is built against libtorch and knows nothing about the runtime's C++ classes: it reaches the endpoints
// through the C function table of slime_bridge.h, whose address the Python side passes in. CUDA tensors are staged
// through host memory (the transports underneath are TCP and RDMA from host memory; between GPUs of one node the NVLink
// operators are the fast path).
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/extension.h>

#include <chrono>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "slime_bridge.h"

namespace {

constexpr int kTimeOut = 402;

class SlimeWork: public c10d::Work {
public:
    struct Part {
        void*      future;  // bridge future
        at::Tensor host;    // buffer the transfer runs on (kept alive)
        at::Tensor device;  // defined for a receive into a CUDA tensor: copied from `host` on completion
    };

    SlimeWork(const SlimeBridge* bridge, int rank, c10d::OpType op, std::vector<Part> parts,
              std::chrono::milliseconds default_timeout):
        c10d::Work(rank, op), bridge_(bridge), parts_(std::move(parts)), default_timeout_(default_timeout)
    {
        future_ = c10::make_intrusive<c10::ivalue::Future>(c10::NoneType::get());
    }

    ~SlimeWork() override
    {
        for (auto& p : parts_)
            if (p.future) bridge_->future_free(p.future);
    }

    bool isCompleted() override
    {
        std::lock_guard<std::mutex> g(mu_);
        if (done_) return true;
        for (auto& p : parts_)
            if (p.future && !bridge_->future_done(p.future)) return false;
        return true;
    }

    bool isSuccess() const override { return done_ && !failed_; }

    bool wait(std::chrono::milliseconds timeout = kNoTimeout) override
    {
        std::lock_guard<std::mutex> g(mu_);
        if (done_) {
            TORCH_CHECK(!failed_, "dlslime backend: the transfer had failed");
            return true;
        }
        const int64_t ms = timeout.count() > 0 ? timeout.count() : default_timeout_.count();
        for (auto& p : parts_) {
            const int status = p.future ? bridge_->future_wait(p.future, ms) : 403;
            if (status != 0) {
                failed_ = true;
                done_   = true;
                auto err = c10::str("dlslime backend: transfer ended with status ", status, status == kTimeOut ? " (timeout)" : "");
                future_->setError(std::make_exception_ptr(std::runtime_error(err)));
                TORCH_CHECK(false, err);
            }
        }
        for (auto& p : parts_)
            if (p.device.defined()) p.device.copy_(p.host, /*non_blocking=*/false);
        done_ = true;
        future_->markCompleted(c10::IValue());
        return true;
    }

    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }

private:
    const SlimeBridge*                      bridge_;
    std::vector<Part>                       parts_;
    std::chrono::milliseconds               default_timeout_;
    std::mutex                              mu_;
    bool                                    done_ = false, failed_ = false;
    c10::intrusive_ptr<c10::ivalue::Future> future_;
};

// The work of endCoalescing: waits for everything issued since startCoalescing.
class GroupWork: public c10d::Work {
public:
    explicit GroupWork(std::vector<c10::intrusive_ptr<c10d::Work>> works): works_(std::move(works)) {}
    bool isCompleted() override
    {
        for (auto& w : works_)
            if (!w->isCompleted()) return false;
        return true;
    }
    bool isSuccess() const override
    {
        for (auto& w : works_)
            if (!w->isSuccess()) return false;
        return true;
    }
    bool wait(std::chrono::milliseconds timeout = kNoTimeout) override
    {
        for (auto& w : works_) w->wait(timeout);
        return true;
    }

private:
    std::vector<c10::intrusive_ptr<c10d::Work>> works_;
};

class SlimeBackend: public c10d::Backend {
public:
    SlimeBackend(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout,
                 const SlimeBridge* bridge, const std::string& transport, const std::string& bind_host):
        c10d::Backend(rank, size), bridge_(bridge), timeout_(timeout.count() > 0 ? timeout : std::chrono::milliseconds(300000))
    {
        TORCH_CHECK(bridge_ && bridge_->version == SLIME_BRIDGE_VERSION, "dlslime backend: bridge table of another version");
        char err[512] = {0};
        for (int peer = 0; peer < size; ++peer) {
            if (peer == rank) continue;
            void* ep = bridge_->endpoint_create(transport.c_str(), bind_host.c_str(), rank, err, sizeof(err));
            TORCH_CHECK(ep != nullptr, "dlslime backend: cannot create an endpoint: ", err);
            eps_[peer] = ep;
            char*             info = bridge_->endpoint_info(ep);
            const std::string text = info ? info : "{}";
            bridge_->free_string(info);
            store->set(key(rank, peer), std::vector<uint8_t>(text.begin(), text.end()));
        }
        for (auto& [peer, ep] : eps_) {
            const std::vector<uint8_t> raw = store->get(key(peer, rank));  // blocks until the peer has published it
            const std::string          text(raw.begin(), raw.end());
            const int                  rc = bridge_->endpoint_connect(ep, text.c_str(), err, sizeof(err));
            TORCH_CHECK(rc == 0, "dlslime backend: connect to rank ", peer, " failed (", rc, "): ", err);
        }
    }

    ~SlimeBackend() override
    {
        for (auto& [peer, ep] : eps_) bridge_->endpoint_destroy(ep);
    }

    const std::string getBackendName() const override { return "dlslime"; }

    std::string transport() const { return eps_.empty() ? std::string("none") : bridge_->endpoint_kind(eps_.begin()->second); }

    void setTimeout(std::chrono::milliseconds timeout) override { timeout_ = timeout; }

    c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dst, int /*tag*/) override
    {
        void*                        ep = endpoint(dst);
        std::vector<SlimeWork::Part> parts;
        for (auto& t : tensors) {
            TORCH_CHECK(t.is_contiguous(), "dlslime backend: tensors must be contiguous");
            at::Tensor host = t.is_cuda() ? t.to(at::kCPU) : t;  // device -> host staging completes before the send is posted
            void*      f    = bridge_->send(ep, reinterpret_cast<uintptr_t>(host.data_ptr()), host.nbytes());
            TORCH_CHECK(f != nullptr, "dlslime backend: send could not be posted");
            parts.push_back({f, host, at::Tensor()});
        }
        return track(c10::make_intrusive<SlimeWork>(bridge_, getRank(), c10d::OpType::SEND, std::move(parts), timeout_));
    }

    c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int src, int /*tag*/) override
    {
        void*                        ep = endpoint(src);
        std::vector<SlimeWork::Part> parts;
        for (auto& t : tensors) {
            TORCH_CHECK(t.is_contiguous(), "dlslime backend: tensors must be contiguous");
            at::Tensor host = t, device;
            if (t.is_cuda()) {
                host   = at::empty(t.sizes(), t.options().device(at::kCPU).pinned_memory(true));
                device = t;
            }
            void* f = bridge_->recv(ep, reinterpret_cast<uintptr_t>(host.data_ptr()), host.nbytes());
            TORCH_CHECK(f != nullptr, "dlslime backend: recv could not be posted");
            parts.push_back({f, host, device});
        }
        return track(c10::make_intrusive<SlimeWork>(bridge_, getRank(), c10d::OpType::RECV, std::move(parts), timeout_));
    }

    void startCoalescing() override
    {
        std::lock_guard<std::mutex> g(mu_);
        coalescing_ = true;
        group_.clear();
    }

    c10::intrusive_ptr<c10d::Work> endCoalescing() override
    {
        std::lock_guard<std::mutex> g(mu_);
        coalescing_ = false;
        auto w      = c10::make_intrusive<GroupWork>(std::move(group_));
        group_.clear();
        return w;
    }

private:
    static std::string key(int from, int to) { return "SLIME_ENDPOINT_" + std::to_string(from) + "_" + std::to_string(to); }

    void* endpoint(int peer)
    {
        auto it = eps_.find(peer);
        TORCH_CHECK(it != eps_.end(), "dlslime backend: rank ", peer, " is not a peer of rank ", getRank());
        return it->second;
    }

    c10::intrusive_ptr<c10d::Work> track(c10::intrusive_ptr<c10d::Work> w)
    {
        std::lock_guard<std::mutex> g(mu_);
        if (coalescing_) group_.push_back(w);
        return w;
    }

    const SlimeBridge*                          bridge_;
    std::chrono::milliseconds                   timeout_;
    std::map<int, void*>                        eps_;
    std::mutex                                  mu_;
    bool                                        coalescing_ = false;
    std::vector<c10::intrusive_ptr<c10d::Work>> group_;
};

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.doc() = "c10d backend 'dlslime' (send / recv over the runtime's endpoints)";
    py::class_<SlimeBackend, c10d::Backend, c10::intrusive_ptr<SlimeBackend>>(m, "SlimeBackend")
        .def("transport", &SlimeBackend::transport);
    m.def(
        "create_backend",
        [](const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, int64_t timeout_ms, uint64_t bridge_table,
           const std::string& transport, const std::string& bind_host) {
            return c10::make_intrusive<SlimeBackend>(store, rank, size, std::chrono::milliseconds(timeout_ms),
                                                     reinterpret_cast<const SlimeBridge*>(bridge_table), transport, bind_host);
        },
        py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout_ms"), py::arg("bridge_table"),
        py::arg("transport") = "", py::arg("bind_host") = "127.0.0.1", py::call_guard<py::gil_scoped_release>());
}
