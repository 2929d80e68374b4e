// Per-operation completion state and the futures handed to callers.
//
// One EndpointOpState owns the outcome of one user-visible operation, however many
// work requests or lanes it was split into: the expected lane mask, the first
// failure status, immediate data, time stamps and the once-only accounting latch.
// Futures share it. wait(timeout_ms) exists on every future; a timeout yields
// TIME_OUT (402) without abandoning the operation.
#pragma once

#include <atomic>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>

#include "core/env.h"
#include "engine/assignment.h"
#include "engine/signal.h"

namespace slime {

struct EndpointOpState {
    std::shared_ptr<DeviceSignal> signal;
    uint32_t                      expected_mask = 1;
    std::atomic<int32_t>          completion_status{SUCCESS};
    std::atomic<int32_t>          imm_data{0};
    std::atomic<uint64_t>         trace_start_ns{0};
    std::atomic<uint64_t>         trace_end_ns{0};
    std::atomic<bool>             obs_completed{false};
    OpCode                        opcode = OpCode::READ;
    uint64_t                      bytes  = 0;
    int                           link_id = -1;

    void fail(int32_t status)
    {
        int32_t ok = SUCCESS;
        completion_status.compare_exchange_strong(ok, status);
    }
};

inline std::shared_ptr<EndpointOpState> make_op_state(uint32_t mask, OpCode op)
{
    auto st           = std::make_shared<EndpointOpState>();
    st->signal        = create_signal(engine_env().bypass_device_signal != 0);
    st->expected_mask = mask;
    st->opcode        = op;
    return st;
}

class DeviceFuture {
public:
    virtual ~DeviceFuture()               = default;
    virtual int32_t wait(int64_t timeout_ms = -1) const = 0;
};

class OpFuture: public DeviceFuture {
public:
    explicit OpFuture(std::shared_ptr<EndpointOpState> st): st_(std::move(st)) {}
    int32_t wait(int64_t timeout_ms = -1) const override
    {
        if (!st_->signal->wait_comm_done_cpu(st_->expected_mask, timeout_ms)) return TIME_OUT;
        const int32_t s = st_->completion_status.load(std::memory_order_acquire);
        // a stream that gave up waiting for this operation ran its consumers without the data
        if (s == SUCCESS && st_->signal->stream_wait_timed_out()) return TIME_OUT;
        return s;
    }
    bool done() const
    {
        return (st_->signal->get_comm_done_mask() & st_->expected_mask) == st_->expected_mask;
    }
    // Makes the stream the operation was submitted with wait (bounded, on the device) for its completion; a no-op for
    // host-only signals.
    // limit_ms > 0 sets the time limit of this wait (default: SLIME_STREAM_WAIT_MS, else 1 s). If the limit runs out,
    // wait() reports TIME_OUT from then on, whatever the transfer itself does later.
    void wait_on_stream(double limit_ms = 0.0) const
    {
        if (limit_ms > 0) st_->signal->set_stream_wait_limit_ns(static_cast<unsigned long long>(limit_ms * 1e6));
        st_->signal->wait_comm_done_on_stream(st_->expected_mask);
    }
    bool stream_wait_timed_out() const { return st_->signal->stream_wait_timed_out(); }
    const std::shared_ptr<EndpointOpState>& state() const { return st_; }

protected:
    std::shared_ptr<EndpointOpState> st_;
};

using SendFuture = OpFuture;
using RecvFuture = OpFuture;

// One-sided operations throw on failure, like the reference's ReadWriteFuture
// (dlslime/csrc/engine/rdma/rdma_future.cpp:49-58 in the reference); a timeout is returned, not thrown.
class ReadWriteFuture: public OpFuture {
public:
    using OpFuture::OpFuture;
    int32_t wait(int64_t timeout_ms = -1) const override
    {
        const int32_t s = OpFuture::wait(timeout_ms);
        if (s != SUCCESS && s != TIME_OUT) throw std::runtime_error("one-sided transfer failed with status " + std::to_string(s));
        return s;
    }
};

class ImmRecvFuture: public OpFuture {
public:
    using OpFuture::OpFuture;
    int32_t  imm_data() const { return st_->imm_data.load(std::memory_order_acquire); }
    bool     time_trace_enabled() const { return st_->trace_start_ns.load() != 0; }
    uint64_t time_trace_start_ns() const { return st_->trace_start_ns.load(); }
    uint64_t time_trace_end_ns() const { return st_->trace_end_ns.load(); }
    uint64_t time_trace_elapsed_ns() const
    {
        const uint64_t s = st_->trace_start_ns.load(), e = st_->trace_end_ns.load();
        return (s != 0 && e >= s) ? e - s : 0;
    }
};

}  // namespace slime
