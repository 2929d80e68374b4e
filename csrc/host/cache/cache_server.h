// DLSlimeCache directory: which slabs of the cache service's registered memory hold
// which peer's assignment batch. It stores no payload; clients move bytes with
// one-sided endpoint writes / reads addressed by the manifests returned here.
// Behaviour matches the reference's CacheServer (dlslime/csrc/cache/cache_server.cpp:10-115
// in the reference): slab sizes in [128 KiB, 1 GiB], optional fixed pool, LIFO slab
// reuse, store-time splitting into slab-sized pieces, versions counting up from 1.
#pragma once

#include <cstdint>
#include <map>
#include <optional>
#include <shared_mutex>
#include <string>
#include <vector>

#include "engine/assignment.h"

namespace slime {
namespace cache {

struct AssignmentManifest {
    std::string           peer_agent_id;
    AssignmentBatch       assignments;
    std::vector<uint64_t> slab_ids;
    uint64_t              version = 0;

    uint64_t total_bytes() const
    {
        uint64_t n = 0;
        for (const auto& a : assignments) n += a.length;
        return n;
    }
};

struct CacheStats {
    uint64_t num_assignment_peers = 0, num_assignment_entries = 0, num_assignments = 0, assignment_bytes = 0;
    uint64_t slab_size = 0, memory_size = 0, num_slabs = 0, used_slabs = 0, free_slabs = 0;
};

class CacheServer {
public:
    static constexpr uint64_t kMinSlabSize       = 128ull << 10;
    static constexpr uint64_t kMaxSlabSize       = 1ull << 30;
    static constexpr uint64_t kDefaultSlabSize   = 256ull << 10;
    static constexpr uint64_t kDefaultMemorySize = 0;

    explicit CacheServer(uint64_t slab_size = kDefaultSlabSize, uint64_t memory_size = kDefaultMemorySize);

    uint64_t slab_size() const { return slab_size_; }
    uint64_t memory_size() const { return memory_size_; }
    uint64_t num_slabs() const { return num_slabs_; }

    AssignmentManifest                store_assignments(const std::string& peer_agent_id, AssignmentBatch batch);
    std::optional<AssignmentManifest> query_assignments(const std::string& peer_agent_id, uint64_t version) const;
    bool                              erase_assignments(const std::string& peer_agent_id, uint64_t version);
    CacheStats                        stats() const;
    void                              clear();

private:
    void reset_free_list();

    const uint64_t slab_size_, memory_size_, num_slabs_;
    mutable std::shared_mutex mu_;
    std::map<std::string, std::map<uint64_t, AssignmentManifest>> entries_;
    std::vector<uint64_t> free_slabs_;    // LIFO: back() is handed out next (fixed pool only)
    uint64_t              next_slab_ = 0;  // growing pool when memory_size == 0
    std::vector<uint64_t> recycled_;      // returned slabs of the growing pool
    uint64_t              used_slabs_   = 0;
    uint64_t              next_version_ = 1;
};

}  // namespace cache
}  // namespace slime
