// Transfer accounting: relaxed atomic counters for the peer as a whole and per link
// (a NIC, an NVLink peer, a TCP connection), read out as one JSON snapshot.
//
// The snapshot keeps the reference's schema (dlslime/csrc/observability/obs.cpp:75-198 in
// the reference: `summary`, `nics[]` with the same field names, `by_op`) and adds `kind`
// ("rdma" | "nvlink" | "tcp") to every link entry so NVLink and TCP bytes are accounted
// the same way as NIC bytes. Gate: DLSLIME_OBS=1, read once; recorders are no-ops otherwise.
#pragma once

#include <atomic>
#include <cstdint>
#include <string>

#include "core/json.hpp"
#include "engine/assignment.h"

namespace slime {
namespace obs {

enum OpIndex : int { OP_READ = 0, OP_WRITE, OP_WRITE_WITH_IMM, OP_SEND, OP_RECV, OP_IMM_RECV, OP_COUNT };
constexpr int kMaxLinks = 64;

const char* op_name(int op);
OpIndex     op_index(OpCode code);

bool enabled();
void set_enabled_for_test(bool on);

// Returns a slot in [0, kMaxLinks) (same name -> same slot) or -1 when disabled / full.
int register_link(const std::string& name, const std::string& kind = "rdma");

// One call per USER operation (not per work request).
void record_submit(int link, OpIndex op, uint64_t n_assign, uint64_t bytes);
void record_complete(int link, OpIndex op, uint64_t bytes);
void record_fail(int link, OpIndex op, uint64_t bytes);
// Posting layer (work requests actually handed to the transport).
void record_post_batch(int link, OpIndex op, uint64_t n_wr, uint64_t bytes);
void record_post_failure(int link, OpIndex op);
void record_cq_error(int link);
void record_mr_register(bool system, uint64_t bytes);
void record_mr_unregister(bool system, uint64_t bytes);
void record_mr_grow(bool system, uint64_t old_bytes, uint64_t new_bytes);

Json snapshot();
void reset_for_test();

}  // namespace obs
}  // namespace slime
