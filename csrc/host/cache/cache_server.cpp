#include "cache/cache_server.h"

#include <algorithm>
#include <mutex>
#include <stdexcept>

namespace slime {
namespace cache {

CacheServer::CacheServer(uint64_t slab_size, uint64_t memory_size):
    slab_size_(slab_size), memory_size_(memory_size), num_slabs_(slab_size ? memory_size / slab_size : 0)
{
    if (slab_size < kMinSlabSize || slab_size > kMaxSlabSize)
        throw std::invalid_argument("slab_size must be in [128K, 1G]");
    if (memory_size % slab_size != 0) throw std::invalid_argument("memory_size must be a multiple of slab_size");
    reset_free_list();
}

void CacheServer::reset_free_list()
{
    free_slabs_.clear();
    recycled_.clear();
    next_slab_  = 0;
    used_slabs_ = 0;
    // lowest id is handed out first
    for (uint64_t i = num_slabs_; i > 0; --i) free_slabs_.push_back(i - 1);
}

AssignmentManifest CacheServer::store_assignments(const std::string& peer_agent_id, AssignmentBatch batch)
{
    if (peer_agent_id.empty()) throw std::invalid_argument("peer_agent_id must not be empty");
    AssignmentBatch pieces;
    split_assign_by_max_length(batch, pieces, slab_size_);

    std::unique_lock<std::shared_mutex> g(mu_);
    const bool fixed = memory_size_ != 0;
    if (fixed && pieces.size() > free_slabs_.size())
        throw std::runtime_error("not enough preallocated cache slabs: need " + std::to_string(pieces.size()) + ", free "
                                 + std::to_string(free_slabs_.size()));
    AssignmentManifest m;
    m.peer_agent_id = peer_agent_id;
    m.version       = next_version_++;
    m.slab_ids.reserve(pieces.size());
    for (auto& a : pieces) {
        uint64_t slab;
        if (fixed) {
            slab = free_slabs_.back();
            free_slabs_.pop_back();
        }
        else if (!recycled_.empty()) {
            slab = recycled_.back();
            recycled_.pop_back();
        }
        else {
            slab = next_slab_++;
        }
        a.source_offset = slab * slab_size_;  // where the bytes live inside the cache region
        m.slab_ids.push_back(slab);
    }
    used_slabs_ += pieces.size();
    m.assignments = std::move(pieces);
    entries_[peer_agent_id][m.version] = m;
    return m;
}

std::optional<AssignmentManifest> CacheServer::query_assignments(const std::string& peer_agent_id, uint64_t version) const
{
    std::shared_lock<std::shared_mutex> g(mu_);
    auto p = entries_.find(peer_agent_id);
    if (p == entries_.end()) return std::nullopt;
    auto v = p->second.find(version);
    if (v == p->second.end()) return std::nullopt;
    return v->second;
}

bool CacheServer::erase_assignments(const std::string& peer_agent_id, uint64_t version)
{
    std::unique_lock<std::shared_mutex> g(mu_);
    auto p = entries_.find(peer_agent_id);
    if (p == entries_.end()) return false;
    auto v = p->second.find(version);
    if (v == p->second.end()) return false;
    auto& dst = memory_size_ != 0 ? free_slabs_ : recycled_;
    for (uint64_t s : v->second.slab_ids) dst.push_back(s);
    used_slabs_ -= v->second.slab_ids.size();
    p->second.erase(v);
    if (p->second.empty()) entries_.erase(p);
    return true;
}

CacheStats CacheServer::stats() const
{
    std::shared_lock<std::shared_mutex> g(mu_);
    CacheStats s;
    s.slab_size   = slab_size_;
    s.memory_size = memory_size_;
    s.num_slabs   = num_slabs_;
    s.used_slabs  = used_slabs_;
    s.free_slabs  = memory_size_ != 0 ? free_slabs_.size() : 0;
    s.num_assignment_peers = entries_.size();
    for (const auto& p : entries_) {
        s.num_assignment_entries += p.second.size();
        for (const auto& v : p.second) {
            s.num_assignments += v.second.assignments.size();
            s.assignment_bytes += v.second.total_bytes();
        }
    }
    return s;
}

void CacheServer::clear()
{
    std::unique_lock<std::shared_mutex> g(mu_);
    entries_.clear();
    next_version_ = 1;
    reset_free_list();
}

}  // namespace cache
}  // namespace slime
