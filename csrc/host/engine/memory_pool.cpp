#include "engine/memory_pool.h"

#include <iterator>

#include <functional>

#include "core/log.h"
#include "obs/obs.h"

namespace slime {

static bool is_system_name(const std::string& n)
{
    return n.rfind("sys.", 0) == 0;
}

int32_t LocalMemoryPool::register_memory_region(uintptr_t addr, uint64_t length, const std::optional<std::string>& name)
{
    std::lock_guard<std::mutex> g(mu_);
    int32_t by_name = -1, by_ptr = -1;
    if (name) {
        auto it = by_name_.find(*name);
        if (it != by_name_.end()) by_name = it->second;
    }
    {
        auto it = by_ptr_.find(addr);
        if (it != by_ptr_.end()) by_ptr = it->second;
    }
    // A name that belongs to one region cannot be pointed at memory that another live region starts at: one of the two
    // would lose its identity (the reference refuses this as well, "registered to diff handle").
    if (by_name >= 0 && by_ptr >= 0 && by_name != by_ptr) return -1;
    int32_t handle = by_name >= 0 ? by_name : by_ptr;
    if (handle >= 0) {
        MemoryRegion& r = regions_[handle];
        // a further name for a region that is already registered is an alias of it (the reference keeps one handle per
        // pointer and lets several names resolve to it, dlslime/csrc/engine/rdma/memory_pool.cpp:27-40 in the reference)
        if (name && by_name_.find(*name) == by_name_.end()) by_name_[*name] = handle;
        if (r.addr == addr && r.length >= length) return handle;  // idempotent
        // same name or same pointer, but moved or grown: register again under the same handle
        if (r.addr != addr) {  // worth a line: two owners using one name in one registry would look exactly like this
            SLIME_LOG_WARN("memory region '", r.name, "' moves from ", reinterpret_cast<void*>(r.addr), " to ",
                           reinterpret_cast<void*>(addr), " under handle ", handle);
            // An automatic name says where the region starts, so it does not survive the move (the region moves under
            // one of its other names): left in place it would collide with the automatic name of whatever is registered
            // at the old address next.
            char was[40];
            snprintf(was, sizeof(was), "auto_0x%llx", static_cast<unsigned long long>(r.addr));
            if (name && *name != was) {
                auto stale = by_name_.find(was);
                if (stale != by_name_.end() && stale->second == handle) {
                    by_name_.erase(stale);
                    if (r.name == was) r.name = *name;
                }
            }
        }
        if (on_unregister) on_unregister(r);
        obs::record_mr_grow(r.system, r.length, length);
        by_ptr_.erase(r.addr);
        r.addr   = addr;
        r.length = length;
        if (on_register) on_register(r);
        by_ptr_[addr] = handle;
        return handle;
    }
    MemoryRegion r;
    r.addr   = addr;
    r.length = length;
    r.alive  = true;
    if (name) {
        r.name = *name;
    }
    else {
        char buf[40];
        snprintf(buf, sizeof(buf), "auto_0x%llx", static_cast<unsigned long long>(addr));
        r.name = buf;
    }
    r.system = is_system_name(r.name);
    if (on_register) on_register(r);
    regions_.push_back(r);
    handle            = static_cast<int32_t>(regions_.size()) - 1;
    by_name_[r.name]  = handle;
    by_ptr_[addr]     = handle;
    obs::record_mr_register(r.system, length);
    return handle;
}

int32_t LocalMemoryPool::unregister_memory_region(int32_t handle)
{
    std::lock_guard<std::mutex> g(mu_);
    if (handle < 0 || handle >= static_cast<int32_t>(regions_.size()) || !regions_[handle].alive) return -1;
    MemoryRegion& r = regions_[handle];
    if (on_unregister) on_unregister(r);
    obs::record_mr_unregister(r.system, r.length);
    for (auto it = by_name_.begin(); it != by_name_.end();)  // the name it was registered under and its aliases
        it = it->second == handle ? by_name_.erase(it) : std::next(it);
    by_ptr_.erase(r.addr);
    r.alive = false;
    return 0;
}

// By name: a region that other names still refer to only loses this name; the last name takes the region with it.
int32_t LocalMemoryPool::unregister_memory_region(const std::string& name)
{
    int32_t h = -1;
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = by_name_.find(name);
        if (it == by_name_.end()) return -1;
        h = it->second;
        std::string other;
        for (const auto& [n, hh] : by_name_)
            if (hh == h && n != name) {
                other = n;
                break;
            }
        if (!other.empty()) {
            by_name_.erase(it);
            if (regions_[static_cast<size_t>(h)].name == name) regions_[static_cast<size_t>(h)].name = other;
            return 0;
        }
    }
    return unregister_memory_region(h);
}

int32_t LocalMemoryPool::get_mr_handle(const std::string& name) const
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = by_name_.find(name);
    return it == by_name_.end() ? -1 : it->second;
}

int32_t LocalMemoryPool::get_mr_handle(uintptr_t addr) const
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = by_ptr_.find(addr);
    return it == by_ptr_.end() ? -1 : it->second;
}

bool LocalMemoryPool::get_mr(int32_t handle, MemoryRegion& out) const
{
    std::lock_guard<std::mutex> g(mu_);
    if (handle < 0 || handle >= static_cast<int32_t>(regions_.size()) || !regions_[handle].alive) return false;
    out = regions_[handle];
    return true;
}

Json LocalMemoryPool::mr_info() const
{
    std::lock_guard<std::mutex> g(mu_);
    Json out = Json::object();
    for (const auto& [name, h] : by_name_) {  // every name, aliases included, describes its region
        const MemoryRegion& r = regions_[static_cast<size_t>(h)];
        if (!r.alive) continue;
        Json e      = Json::object();
        e["handle"] = static_cast<long long>(h);
        e["addr"]   = static_cast<unsigned long long>(r.addr);
        e["rkey"]   = static_cast<unsigned long long>(r.rkey);
        e["length"] = static_cast<unsigned long long>(r.length);
        out[name]   = e;
    }
    return out;
}

size_t LocalMemoryPool::live_count() const
{
    std::lock_guard<std::mutex> g(mu_);
    size_t n = 0;
    for (const auto& r : regions_) n += r.alive ? 1 : 0;
    return n;
}

int32_t RemoteMemoryPool::register_remote_memory_region(const std::string& name, const Json& info)
{
    MemoryRegion r;
    r.name   = name;
    r.addr   = static_cast<uintptr_t>(info["addr"].as_uint());
    r.length = info["length"].as_uint();
    r.rkey   = info["rkey"].as_uint();
    r.alive  = true;
    std::lock_guard<std::mutex> g(mu_);
    auto it = by_name_.find(name);
    if (it != by_name_.end()) {
        MemoryRegion& cur = regions_[it->second];
        if (cur.addr != r.addr || cur.length != r.length || cur.rkey != r.rkey || !cur.alive) cur = r;
        return it->second;
    }
    regions_.push_back(r);
    by_name_[name] = static_cast<int32_t>(regions_.size()) - 1;
    return static_cast<int32_t>(regions_.size()) - 1;
}

int32_t RemoteMemoryPool::register_remote_memory_region(uintptr_t addr, uint64_t length, uint64_t rkey)
{
    char buf[40];
    snprintf(buf, sizeof(buf), "remote_0x%llx", static_cast<unsigned long long>(addr));
    Json info      = Json::object();
    info["addr"]   = static_cast<unsigned long long>(addr);
    info["length"] = static_cast<unsigned long long>(length);
    info["rkey"]   = static_cast<unsigned long long>(rkey);
    return register_remote_memory_region(buf, info);
}

int32_t RemoteMemoryPool::unregister_remote_memory_region(const std::string& name)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = by_name_.find(name);
    if (it == by_name_.end()) return -1;
    regions_[it->second].alive = false;
    by_name_.erase(it);
    return 0;
}

int32_t RemoteMemoryPool::get_remote_mr_handle(const std::string& name) const
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = by_name_.find(name);
    return it == by_name_.end() ? -1 : it->second;
}

bool RemoteMemoryPool::get_remote_mr(int32_t handle, MemoryRegion& out) const
{
    std::lock_guard<std::mutex> g(mu_);
    if (handle < 0 || handle >= static_cast<int32_t>(regions_.size()) || !regions_[handle].alive) return false;
    out = regions_[handle];
    return true;
}

Json RemoteMemoryPool::remote_mr_info() const
{
    std::lock_guard<std::mutex> g(mu_);
    Json out = Json::object();
    for (size_t h = 0; h < regions_.size(); ++h) {
        const MemoryRegion& r = regions_[h];
        if (!r.alive) continue;
        Json e      = Json::object();
        e["handle"] = static_cast<long long>(h);
        e["addr"]   = static_cast<unsigned long long>(r.addr);
        e["rkey"]   = static_cast<unsigned long long>(r.rkey);
        e["length"] = static_cast<unsigned long long>(r.length);
        out[r.name] = e;
    }
    return out;
}

}  // namespace slime
