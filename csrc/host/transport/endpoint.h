// The transport-independent endpoint interface: one object per peer connection that
// owns the local / remote memory-region registries and offers one-sided read / write /
// write-with-immediate, immediate receive and two-sided send / recv, all returning
// futures. TCP (CPU ranks), RDMA RC verbs and the Ascend stub implement it; the RPC
// session, PeerAgent and the torch backend are written against it. Method names and tuple
// orders follow the reference's RDMAEndpoint (dlslime/csrc/engine/rdma/rdma_endpoint.h:203-259
// in the reference).
#pragma once

#include <memory>
#include <string>
#include <vector>

#include "core/json.hpp"
#include "engine/assignment.h"
#include "engine/future.h"
#include "engine/memory_pool.h"

namespace slime {

class Endpoint {
public:
    virtual ~Endpoint() = default;

    virtual std::string kind() const = 0;  // "tcp" | "rdma" | "ascend"
    virtual Json        endpoint_info()                      = 0;
    virtual int         connect(const Json& remote_info)     = 0;
    virtual bool        connected() const                    = 0;

    // Memory regions. A name registers / looks up in the local pool; the returned handle is what
    // assignment tuples carry. Remote regions are registered from the owner's mr_info entry.
    virtual int32_t register_memory_region(const std::string& name, uintptr_t ptr, uintptr_t offset, size_t length)
    {
        return local_pool_->register_memory_region(ptr + offset, length, name);
    }
    virtual int32_t register_memory_region(uintptr_t ptr, uintptr_t offset, size_t length)
    {
        return local_pool_->register_memory_region(ptr + offset, length, std::nullopt);
    }
    virtual int32_t register_remote_memory_region(const std::string& name, const Json& info)
    {
        return remote_pool_->register_remote_memory_region(name, info);
    }
    Json mr_info() const { return local_pool_->mr_info(); }

    virtual std::shared_ptr<ReadWriteFuture> read(const std::vector<assign_tuple_t>& assign, void* stream = nullptr) = 0;
    virtual std::shared_ptr<ReadWriteFuture> write(const std::vector<assign_tuple_t>& assign, void* stream = nullptr) = 0;
    virtual std::shared_ptr<ReadWriteFuture> write_with_imm(const std::vector<assign_tuple_t>& assign, int32_t imm_data,
                                                            void* stream = nullptr) = 0;
    virtual std::shared_ptr<ImmRecvFuture>   imm_recv(void* stream = nullptr)       = 0;
    virtual std::shared_ptr<SendFuture>      send(const chunk_tuple_t& chunk, void* stream = nullptr) = 0;
    virtual std::shared_ptr<RecvFuture>      recv(const chunk_tuple_t& chunk, void* stream = nullptr) = 0;

    // Fails every operation in flight with FAILED (403), wakes every waiter, releases resources. Idempotent.
    virtual void shutdown()   = 0;
    virtual void cancel_all() = 0;
    virtual int  process() { return 0; }  // one turn of the progress engine, for callers that drive it themselves

    // Endpoints of one agent may share a registry so that a region has one handle agent-wide.
    void set_local_pool(std::shared_ptr<LocalMemoryPool> pool) { local_pool_ = std::move(pool); }
    const std::shared_ptr<LocalMemoryPool>&  local_pool() const { return local_pool_; }
    const std::shared_ptr<RemoteMemoryPool>& remote_pool() const { return remote_pool_; }

protected:
    std::shared_ptr<LocalMemoryPool>  local_pool_  = std::make_shared<LocalMemoryPool>();
    std::shared_ptr<RemoteMemoryPool> remote_pool_ = std::make_shared<RemoteMemoryPool>();
};

}  // namespace slime
