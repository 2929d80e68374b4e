#include "obs/obs.h"

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace slime {
namespace obs {

namespace {

struct alignas(64) PeerCounters {
    std::atomic<uint64_t> assign_total{0}, batch_total{0}, submitted_bytes{0}, completed_bytes{0}, failed_bytes{0};
    std::atomic<int64_t>  pending_ops{0};
    std::atomic<uint64_t> error_total{0};
    std::atomic<uint64_t> user_mr_count{0}, user_mr_bytes{0}, sys_mr_count{0}, sys_mr_bytes{0};
    std::atomic<int64_t>  pending_by_op[OP_COUNT];
};

struct alignas(64) LinkCounters {
    std::atomic<uint64_t> assign[OP_COUNT], batch[OP_COUNT], submitted_bytes[OP_COUNT], completed_bytes[OP_COUNT],
        failed_bytes[OP_COUNT], errors[OP_COUNT], post_batch[OP_COUNT], post_wr[OP_COUNT], post_bytes[OP_COUNT],
        post_failures[OP_COUNT];
    std::atomic<int64_t>  pending[OP_COUNT];
    std::atomic<uint64_t> cq_errors{0};
    char                  name[64];
    char                  kind[16];
    std::atomic<bool>     active{false};
};

PeerCounters     g_peer;
LinkCounters     g_links[kMaxLinks];
std::atomic<int> g_link_count{0};
std::mutex       g_register_mu;
std::atomic<int> g_enabled{-1};  // -1 = not read yet

inline bool valid(int link)
{
    return link >= 0 && link < kMaxLinks;
}

void zero_link(LinkCounters& l)
{
    for (int op = 0; op < OP_COUNT; ++op) {
        l.assign[op] = l.batch[op] = l.submitted_bytes[op] = l.completed_bytes[op] = l.failed_bytes[op] = 0;
        l.errors[op] = l.post_batch[op] = l.post_wr[op] = l.post_bytes[op] = l.post_failures[op] = 0;
        l.pending[op] = 0;
    }
    l.cq_errors = 0;
}

}  // namespace

const char* op_name(int op)
{
    static const char* names[OP_COUNT] = {"read", "write", "write_with_imm", "send", "recv", "imm_recv"};
    return (op >= 0 && op < OP_COUNT) ? names[op] : "unknown";
}

OpIndex op_index(OpCode code)
{
    switch (code) {
        case OpCode::READ: return OP_READ;
        case OpCode::WRITE: return OP_WRITE;
        case OpCode::WRITE_WITH_IMM: return OP_WRITE_WITH_IMM;
        case OpCode::SEND:
        case OpCode::SEND_WITH_IMM: return OP_SEND;
        case OpCode::RECV: return OP_RECV;
    }
    return OP_READ;
}

bool enabled()
{
    int e = g_enabled.load(std::memory_order_relaxed);
    if (e < 0) {
        const char* v = std::getenv("DLSLIME_OBS");
        e             = (v != nullptr && std::strcmp(v, "1") == 0) ? 1 : 0;
        g_enabled.store(e, std::memory_order_relaxed);
    }
    return e == 1;
}

void set_enabled_for_test(bool on)
{
    g_enabled.store(on ? 1 : 0);
}

int register_link(const std::string& name, const std::string& kind)
{
    if (!enabled()) return -1;
    std::lock_guard<std::mutex> g(g_register_mu);
    const int n = g_link_count.load(std::memory_order_acquire);
    for (int i = 0; i < n; ++i)
        if (g_links[i].active.load() && name == g_links[i].name) return i;
    if (n >= kMaxLinks) return -1;
    LinkCounters& l = g_links[n];
    zero_link(l);
    std::strncpy(l.name, name.c_str(), sizeof(l.name) - 1);
    l.name[sizeof(l.name) - 1] = 0;
    std::strncpy(l.kind, kind.c_str(), sizeof(l.kind) - 1);
    l.kind[sizeof(l.kind) - 1] = 0;
    l.active.store(true, std::memory_order_release);
    g_link_count.store(n + 1, std::memory_order_release);  // published last: readers see a complete slot
    return n;
}

void record_submit(int link, OpIndex op, uint64_t n_assign, uint64_t bytes)
{
    if (!enabled()) return;
    g_peer.assign_total.fetch_add(n_assign, std::memory_order_relaxed);
    g_peer.batch_total.fetch_add(1, std::memory_order_relaxed);
    g_peer.submitted_bytes.fetch_add(bytes, std::memory_order_relaxed);
    g_peer.pending_ops.fetch_add(1, std::memory_order_relaxed);
    g_peer.pending_by_op[op].fetch_add(1, std::memory_order_relaxed);
    if (valid(link)) {
        LinkCounters& l = g_links[link];
        l.assign[op].fetch_add(n_assign, std::memory_order_relaxed);
        l.batch[op].fetch_add(1, std::memory_order_relaxed);
        l.submitted_bytes[op].fetch_add(bytes, std::memory_order_relaxed);
        l.pending[op].fetch_add(1, std::memory_order_relaxed);
    }
}

void record_complete(int link, OpIndex op, uint64_t bytes)
{
    if (!enabled()) return;
    g_peer.completed_bytes.fetch_add(bytes, std::memory_order_relaxed);
    g_peer.pending_ops.fetch_sub(1, std::memory_order_relaxed);
    g_peer.pending_by_op[op].fetch_sub(1, std::memory_order_relaxed);
    if (valid(link)) {
        g_links[link].completed_bytes[op].fetch_add(bytes, std::memory_order_relaxed);
        g_links[link].pending[op].fetch_sub(1, std::memory_order_relaxed);
    }
}

void record_fail(int link, OpIndex op, uint64_t bytes)
{
    if (!enabled()) return;
    g_peer.failed_bytes.fetch_add(bytes, std::memory_order_relaxed);
    g_peer.error_total.fetch_add(1, std::memory_order_relaxed);
    g_peer.pending_ops.fetch_sub(1, std::memory_order_relaxed);
    g_peer.pending_by_op[op].fetch_sub(1, std::memory_order_relaxed);
    if (valid(link)) {
        g_links[link].failed_bytes[op].fetch_add(bytes, std::memory_order_relaxed);
        g_links[link].errors[op].fetch_add(1, std::memory_order_relaxed);
        g_links[link].pending[op].fetch_sub(1, std::memory_order_relaxed);
    }
}

void record_post_batch(int link, OpIndex op, uint64_t n_wr, uint64_t bytes)
{
    if (!enabled() || !valid(link)) return;
    g_links[link].post_batch[op].fetch_add(1, std::memory_order_relaxed);
    g_links[link].post_wr[op].fetch_add(n_wr, std::memory_order_relaxed);
    g_links[link].post_bytes[op].fetch_add(bytes, std::memory_order_relaxed);
}

void record_post_failure(int link, OpIndex op)
{
    if (!enabled() || !valid(link)) return;
    g_links[link].post_failures[op].fetch_add(1, std::memory_order_relaxed);
}

void record_cq_error(int link)
{
    if (!enabled() || !valid(link)) return;
    g_links[link].cq_errors.fetch_add(1, std::memory_order_relaxed);
}

void record_mr_register(bool system, uint64_t bytes)
{
    if (!enabled()) return;
    (system ? g_peer.sys_mr_count : g_peer.user_mr_count).fetch_add(1, std::memory_order_relaxed);
    (system ? g_peer.sys_mr_bytes : g_peer.user_mr_bytes).fetch_add(bytes, std::memory_order_relaxed);
}

void record_mr_unregister(bool system, uint64_t bytes)
{
    if (!enabled()) return;
    (system ? g_peer.sys_mr_count : g_peer.user_mr_count).fetch_sub(1, std::memory_order_relaxed);
    (system ? g_peer.sys_mr_bytes : g_peer.user_mr_bytes).fetch_sub(bytes, std::memory_order_relaxed);
}

void record_mr_grow(bool system, uint64_t old_bytes, uint64_t new_bytes)
{
    if (!enabled()) return;
    auto& b = system ? g_peer.sys_mr_bytes : g_peer.user_mr_bytes;
    b.fetch_sub(old_bytes, std::memory_order_relaxed);
    b.fetch_add(new_bytes, std::memory_order_relaxed);
}

Json snapshot()
{
    Json out = Json::object();
    if (!enabled()) {
        out["enabled"] = false;
        return out;
    }
    auto U = [](const std::atomic<uint64_t>& a) { return Json(static_cast<unsigned long long>(a.load(std::memory_order_relaxed))); };
    auto I = [](const std::atomic<int64_t>& a) { return Json(static_cast<long long>(a.load(std::memory_order_relaxed))); };
    Json s                     = Json::object();
    s["assign_total"]          = U(g_peer.assign_total);
    s["batch_total"]           = U(g_peer.batch_total);
    s["submitted_bytes_total"] = U(g_peer.submitted_bytes);
    s["completed_bytes_total"] = U(g_peer.completed_bytes);
    s["failed_bytes_total"]    = U(g_peer.failed_bytes);
    s["pending_ops"]           = I(g_peer.pending_ops);
    s["error_total"]           = U(g_peer.error_total);
    s["user_mr_count"]         = U(g_peer.user_mr_count);
    s["user_mr_bytes"]         = U(g_peer.user_mr_bytes);
    s["sys_mr_count"]          = U(g_peer.sys_mr_count);
    s["sys_mr_bytes"]          = U(g_peer.sys_mr_bytes);
    s["mr_count"]              = s["user_mr_count"];
    s["mr_bytes"]              = s["user_mr_bytes"];
    Json pend                  = Json::object();
    for (int op = 0; op < OP_COUNT; ++op) pend[op_name(op)] = I(g_peer.pending_by_op[op]);
    s["pending_by_op"] = pend;

    Json      links = Json::array();
    const int n     = g_link_count.load(std::memory_order_acquire);
    for (int i = 0; i < n && i < kMaxLinks; ++i) {
        LinkCounters& l = g_links[i];
        if (!l.active.load(std::memory_order_acquire)) continue;
        uint64_t t[10] = {0};
        int64_t  pending = 0;
        Json     by_op   = Json::object();
        for (int op = 0; op < OP_COUNT; ++op) {
            const uint64_t v[10] = {l.assign[op].load(), l.batch[op].load(), l.submitted_bytes[op].load(),
                                    l.completed_bytes[op].load(), l.failed_bytes[op].load(), l.errors[op].load(),
                                    l.post_batch[op].load(), l.post_wr[op].load(), l.post_bytes[op].load(),
                                    l.post_failures[op].load()};
            const int64_t  p     = l.pending[op].load();
            for (int k = 0; k < 10; ++k) t[k] += v[k];
            pending += p;
            if (v[0] || v[1] || v[2] || v[3]) {
                Json o               = Json::object();
                o["assign"]          = static_cast<unsigned long long>(v[0]);
                o["batch"]           = static_cast<unsigned long long>(v[1]);
                o["submitted_bytes"] = static_cast<unsigned long long>(v[2]);
                o["completed_bytes"] = static_cast<unsigned long long>(v[3]);
                o["failed_bytes"]    = static_cast<unsigned long long>(v[4]);
                o["pending"]         = static_cast<long long>(p);
                o["errors"]          = static_cast<unsigned long long>(v[5]);
                o["post_batch"]      = static_cast<unsigned long long>(v[6]);
                o["post_wr"]         = static_cast<unsigned long long>(v[7]);
                o["post_bytes"]      = static_cast<unsigned long long>(v[8]);
                o["post_failures"]   = static_cast<unsigned long long>(v[9]);
                by_op[op_name(op)]   = o;
            }
        }
        Json e                     = Json::object();
        e["nic"]                   = std::string(l.name);
        e["kind"]                  = std::string(l.kind);
        e["nic_bdf"]               = "";
        e["assign_total"]          = static_cast<unsigned long long>(t[0]);
        e["batch_total"]           = static_cast<unsigned long long>(t[1]);
        e["submitted_bytes_total"] = static_cast<unsigned long long>(t[2]);
        e["completed_bytes_total"] = static_cast<unsigned long long>(t[3]);
        e["failed_bytes_total"]    = static_cast<unsigned long long>(t[4]);
        e["pending_ops"]           = static_cast<long long>(pending);
        e["error_total"]           = static_cast<unsigned long long>(t[5]);
        e["post_batch_total"]      = static_cast<unsigned long long>(t[6]);
        e["post_wr_total"]         = static_cast<unsigned long long>(t[7]);
        e["post_bytes_total"]      = static_cast<unsigned long long>(t[8]);
        e["post_failures_total"]   = static_cast<unsigned long long>(t[9]);
        e["cq_errors_total"]       = static_cast<unsigned long long>(l.cq_errors.load());
        if (by_op.size() > 0) e["by_op"] = by_op;
        links.push_back(e);
    }
    out["enabled"] = true;
    out["summary"] = s;
    out["nics"]    = links;
    return out;
}

void reset_for_test()
{
    std::lock_guard<std::mutex> g(g_register_mu);
    g_peer.assign_total = g_peer.batch_total = g_peer.submitted_bytes = g_peer.completed_bytes = g_peer.failed_bytes = 0;
    g_peer.pending_ops = 0;
    g_peer.error_total = 0;
    g_peer.user_mr_count = g_peer.user_mr_bytes = g_peer.sys_mr_count = g_peer.sys_mr_bytes = 0;
    for (int op = 0; op < OP_COUNT; ++op) g_peer.pending_by_op[op] = 0;
    const int n = g_link_count.load();
    for (int i = 0; i < n; ++i) {
        zero_link(g_links[i]);
        g_links[i].active.store(false);
    }
    g_link_count.store(0);
}

}  // namespace obs
}  // namespace slime
