// Registry of local and remote memory regions: names <-> integer handles <-> extents.
//
// Semantics follow the reference's RDMA pools (dlslime/csrc/engine/rdma/memory_pool.cpp:18-221,
// remote_memory_pool.h:26-95 in the reference): registering the same pointer again
// returns the same handle, a region that grew is re-registered in place, names starting
// with "sys." are accounted as system regions, unregistering frees the name and the
// pointer key but handles are never reused. Transport-specific keys (an rkey, an IPC
// handle, ...) ride along as opaque 64-bit values and JSON extras.
#pragma once

#include <cstdint>
#include <functional>
#include <mutex>
#include <optional>
#include <string>
#include <unordered_map>
#include <vector>

#include "core/json.hpp"

namespace slime {

struct MemoryRegion {
    std::string name;
    uintptr_t   addr   = 0;
    uint64_t    length = 0;
    uint64_t    rkey   = 0;  // transport key published to peers
    uint64_t    lkey   = 0;
    uint64_t    opaque = 0;  // transport object behind the keys (for example the verbs memory region)
    bool        alive  = false;
    bool        system = false;

    bool contains(uint64_t offset, uint64_t len) const { return alive && offset <= length && len <= length - offset; }
};

class LocalMemoryPool {
public:
    // Hook invoked under the pool lock when a region is (re-)registered / dropped; the transport
    // fills rkey / lkey (for example by ibv_reg_mr). May be empty.
    std::function<void(MemoryRegion&)>       on_register;
    std::function<void(const MemoryRegion&)> on_unregister;

    int32_t register_memory_region(uintptr_t addr, uint64_t length, const std::optional<std::string>& name = std::nullopt);
    int32_t unregister_memory_region(int32_t handle);
    int32_t unregister_memory_region(const std::string& name);
    int32_t get_mr_handle(const std::string& name) const;
    int32_t get_mr_handle(uintptr_t addr) const;
    bool    get_mr(int32_t handle, MemoryRegion& out) const;
    Json    mr_info() const;  // {name: {handle, addr, rkey, length}}
    size_t  live_count() const;

private:
    mutable std::mutex                       mu_;
    std::vector<MemoryRegion>                regions_;
    std::unordered_map<std::string, int32_t> by_name_;
    std::unordered_map<uintptr_t, int32_t>   by_ptr_;
};

class RemoteMemoryPool {
public:
    // info = {addr, length, rkey, ...}; an existing name is updated in place when it changed.
    int32_t register_remote_memory_region(const std::string& name, const Json& info);
    int32_t register_remote_memory_region(uintptr_t addr, uint64_t length, uint64_t rkey);
    int32_t unregister_remote_memory_region(const std::string& name);
    int32_t get_remote_mr_handle(const std::string& name) const;
    bool    get_remote_mr(int32_t handle, MemoryRegion& out) const;
    Json    remote_mr_info() const;

private:
    mutable std::mutex                       mu_;
    std::vector<MemoryRegion>                regions_;
    std::unordered_map<std::string, int32_t> by_name_;
};

}  // namespace slime
