// The transfer descriptor shared by every endpoint, and its splitters.
//
// For BOTH read and write, target_offset is the offset inside the REMOTE region and
// source_offset the offset inside the LOCAL region (the behaviour of the reference's
// data path, dlslime/csrc/engine/rdma/rdma_channel.cpp:322-341 in the reference).
// Tuple forms used by the Python API:
//   assign tuple        (local_handle, remote_handle, target_offset, source_offset, length)
//   named assign tuple  (local_name,   remote_name,   target_offset, source_offset, length)
//   chunk tuple         (data_ptr, offset, length)               for send / recv
#pragma once

#include <algorithm>
#include <cstdint>
#include <string>
#include <tuple>
#include <vector>

#include "core/json.hpp"

namespace slime {

enum class OpCode : uint8_t { READ = 0, WRITE = 1, SEND = 2, RECV = 3, SEND_WITH_IMM = 4, WRITE_WITH_IMM = 5 };

inline const char* opcode_name(OpCode op)
{
    switch (op) {
        case OpCode::READ: return "read";
        case OpCode::WRITE: return "write";
        case OpCode::SEND: return "send";
        case OpCode::RECV: return "recv";
        case OpCode::SEND_WITH_IMM: return "send_with_imm";
        case OpCode::WRITE_WITH_IMM: return "write_with_imm";
    }
    return "unknown";
}

// Completion codes surfaced by futures.
enum StatusCode : int32_t {
    SUCCESS                   = 0,
    ASSIGNMENT_BATCH_OVERFLOW = 400,
    UNKNOWN_OPCODE            = 401,
    TIME_OUT                  = 402,
    FAILED                    = 403,
};

using assign_tuple_t       = std::tuple<uintptr_t, uintptr_t, uint64_t, uint64_t, size_t>;
using chunk_tuple_t        = std::tuple<uintptr_t, uint64_t, size_t>;
using named_assign_tuple_t = std::tuple<std::string, std::string, uint64_t, uint64_t, size_t>;

struct alignas(64) Assignment {
    uintptr_t mr_key{};         // local region handle (or pointer key)
    uintptr_t remote_mr_key{};  // remote region handle
    uint64_t  target_offset{};  // byte offset in the remote region
    uint64_t  source_offset{};  // byte offset in the local region
    uint64_t  length{};

    Assignment() = default;
    Assignment(uintptr_t key, uint64_t target_off, uint64_t source_off, uint64_t len):
        mr_key(key), remote_mr_key(key), target_offset(target_off), source_offset(source_off), length(len)
    {
    }
    Assignment(uintptr_t key, uintptr_t remote_key, uint64_t target_off, uint64_t source_off, uint64_t len):
        mr_key(key), remote_mr_key(remote_key), target_offset(target_off), source_offset(source_off), length(len)
    {
    }
    explicit Assignment(const assign_tuple_t& t):
        mr_key(std::get<0>(t)), remote_mr_key(std::get<1>(t)), target_offset(std::get<2>(t)), source_offset(std::get<3>(t)),
        length(std::get<4>(t))
    {
    }

    Json to_json() const
    {
        Json j = Json::object();
        j["mr_key"]        = static_cast<unsigned long long>(mr_key);
        j["remote_mr_key"] = static_cast<unsigned long long>(remote_mr_key);
        j["target_offset"] = static_cast<unsigned long long>(target_offset);
        j["source_offset"] = static_cast<unsigned long long>(source_offset);
        j["length"]        = static_cast<unsigned long long>(length);
        return j;
    }
    std::string dump() const { return to_json().dump(); }
};

using AssignmentBatch = std::vector<Assignment>;

// Every assignment longer than max_length becomes consecutive pieces of at most max_length.
void split_assign_by_max_length(const AssignmentBatch& in, AssignmentBatch& out, size_t max_length);
// Consecutive groups of `step` assignments.
void split_assign_by_step(const AssignmentBatch& in, std::vector<AssignmentBatch>& out, size_t step);
// At most nstep groups of equal size (the last may be shorter).
void nsplit_assign_by_step(const AssignmentBatch& in, std::vector<AssignmentBatch>& out, size_t nstep);

}  // namespace slime
