// Completion signalling between the submitting thread, the progress / completion
// threads and (for device buffers) the CUDA stream.
//
// DeviceSignal mirrors the reference's interface (dlslime/csrc/device/signal.h:7-27 in the
// reference): a "GPU ready" flag that gates posting, and a "communication done" bit mask
// with one bit per lane (queue pair / connection) that completion callbacks OR into.
// HostSignal is the CPU implementation. For CUDA streams the same roles are played by the
// flag kernels of libslime_cuda (slime_signal_flag_kernel / slime_wait_flag_kernel, bounded
// waits) on a mapped host word, attached through StreamHooks so this library needs no CUDA.
#pragma once

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <memory>
#include <mutex>

#include "core/ring.h"

namespace slime {

class DeviceSignal {
public:
    virtual ~DeviceSignal() = default;
    virtual void     init()                                         = 0;
    virtual void     record_gpu_ready()                             = 0;
    virtual bool     is_gpu_ready() const                           = 0;
    virtual uint32_t get_comm_done_mask() const                     = 0;
    virtual void     set_comm_done(int lane)                        = 0;
    virtual void     bind_stream(void* stream)                      = 0;
    virtual void     wait_comm_done_on_stream(uint32_t mask)        = 0;
    // Blocks until (done & mask) == mask or force_complete(); timeout_ms < 0 waits for ever.
    // Returns false on timeout.
    virtual bool wait_comm_done_cpu(uint32_t mask, int64_t timeout_ms = -1) = 0;
    virtual void force_complete()                                   = 0;
    virtual void reset_all()                                        = 0;
};

// Hooks that let a CUDA-aware layer order transfers against a stream without linking CUDA here.
struct StreamHooks {
    // enqueue "write 1 to *flag" on the stream (buffer is ready once it executes)
    std::function<void(void* stream, std::atomic<uint32_t>* flag)> record_ready;
    // make the stream wait until (*done & mask) == mask
    std::function<void(void* stream, std::atomic<uint32_t>* done, uint32_t mask)> wait_done;
};

inline StreamHooks& stream_hooks()
{
    static StreamHooks hooks;
    return hooks;
}

class HostSignal final: public DeviceSignal {
public:
    void init() override { reset_all(); }
    void record_gpu_ready() override
    {
        if (stream_ != nullptr && stream_hooks().record_ready) {
            stream_hooks().record_ready(stream_, &gpu_ready_);
            return;
        }
        gpu_ready_.store(1, std::memory_order_release);
    }
    bool     is_gpu_ready() const override { return gpu_ready_.load(std::memory_order_acquire) != 0; }
    uint32_t get_comm_done_mask() const override { return done_.load(std::memory_order_acquire); }
    void     set_comm_done(int lane) override
    {
        done_.fetch_or(1u << lane, std::memory_order_acq_rel);
        notify();
    }
    void bind_stream(void* stream) override { stream_ = stream; }
    void wait_comm_done_on_stream(uint32_t mask) override
    {
        if (stream_ != nullptr && stream_hooks().wait_done) stream_hooks().wait_done(stream_, &done_, mask);
    }
    bool wait_comm_done_cpu(uint32_t mask, int64_t timeout_ms = -1) override
    {
        auto satisfied = [&] { return forced_.load(std::memory_order_acquire) || (done_.load(std::memory_order_acquire) & mask) == mask; };
        // short spin for the latency-critical case, then sleep on the condition variable
        for (int i = 0; i < 2000; ++i) {
            if (satisfied()) return true;
            cpu_pause();
        }
        std::unique_lock<std::mutex> g(mu_);
        if (timeout_ms < 0) {
            cv_.wait(g, satisfied);
            return true;
        }
        return cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), satisfied);
    }
    void force_complete() override
    {
        forced_.store(true, std::memory_order_release);
        notify();
    }
    void reset_all() override
    {
        gpu_ready_.store(0, std::memory_order_relaxed);
        done_.store(0, std::memory_order_relaxed);
        forced_.store(false, std::memory_order_release);
    }

private:
    void notify()
    {
        std::lock_guard<std::mutex> g(mu_);
        cv_.notify_all();
    }
    std::atomic<uint32_t>   gpu_ready_{0};
    std::atomic<uint32_t>   done_{0};
    std::atomic<bool>       forced_{false};
    void*                   stream_ = nullptr;
    std::mutex              mu_;
    std::condition_variable cv_;
};

inline std::shared_ptr<DeviceSignal> create_signal(bool /*bypass*/ = true)
{
    auto s = std::make_shared<HostSignal>();
    s->init();
    return s;
}

}  // namespace slime
