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
#include <cstdlib>
#include <functional>
#include <memory>
#include <mutex>
#include <vector>

#include "core/nvtx.h"
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
    // True once a stream-ordered wait gave up at its time limit: what was queued behind it on the stream ran without
    // the transferred bytes, so the operation must not be reported as a success.
    virtual bool     stream_wait_timed_out() const { return false; }
    // Time limit of the stream-ordered wait in nanoseconds (0 = the process default, SLIME_STREAM_WAIT_MS or 1 s).
    virtual void     set_stream_wait_limit_ns(unsigned long long) {}
    // Blocks until (done & mask) == mask or force_complete(); timeout_ms < 0 waits for ever.
    // Returns false on timeout.
    virtual bool wait_comm_done_cpu(uint32_t mask, int64_t timeout_ms = -1) = 0;
    virtual void force_complete()                                   = 0;
    virtual void reset_all()                                        = 0;
};

// Hooks that let a CUDA-aware layer order transfers against a stream without linking CUDA here. They are plain C
// function pointers (the kernel library exports matching functions); words are 64-bit and live in pinned host
// memory that the device can address.
struct StreamHooks {
    int (*alloc_words)(unsigned long long n_words, void** host, void** dev)                         = nullptr;
    int (*free_words)(void* host)                                                                   = nullptr;
    // enqueue on `stream`: *word = value (release at system scope): "the buffer is ready once this has run"
    int (*record_value)(void* stream, void* dev_word, unsigned long long value)                     = nullptr;
    // enqueue on `stream`: wait (bounded) until (*word & mask) == mask; when the limit runs out first, store 1 to
    // *timeout_word (release at system scope) and return
    int (*wait_mask)(void* stream, void* dev_word, unsigned long long mask, unsigned long long limit_ns,
                     void* dev_timeout_word) = nullptr;
    bool installed() const { return alloc_words && free_words && record_value && wait_mask; }
};
inline StreamHooks& stream_hooks()
{
    static StreamHooks hooks;
    return hooks;
}

class HostSignal final: public DeviceSignal {
public:
    void init() override { reset_all(); }
    void record_gpu_ready() override { gpu_ready_.store(1, std::memory_order_release); }
    bool     is_gpu_ready() const override { return gpu_ready_.load(std::memory_order_acquire) != 0; }
    uint32_t get_comm_done_mask() const override { return done_.load(std::memory_order_acquire); }
    void     set_comm_done(int lane) override
    {
        done_.fetch_or(1u << lane, std::memory_order_acq_rel);
        notify();
    }
    void bind_stream(void* stream) override { stream_ = stream; }
    void wait_comm_done_on_stream(uint32_t) override {}  // no device-visible words: use MappedSignal for stream ordering
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

// Pool of device-addressable words (four per signal: ready, done, wait-timed-out, spare), allocated from the hooks in
// chunks and recycled.
class MappedWordPool {
public:
    struct Pair {
        std::atomic<unsigned long long>* host = nullptr;  // [4]
        void*                            dev  = nullptr;  // device address of host[0]
    };
    static MappedWordPool& get()
    {
        static MappedWordPool* p = new MappedWordPool();  // pinned memory is returned to the driver at process exit
        return *p;
    }
    bool acquire(Pair& out)
    {
        std::lock_guard<std::mutex> g(mu_);
        if (free_.empty()) {
            constexpr unsigned long long kPairs = 128;
            void *h = nullptr, *d = nullptr;
            if (!stream_hooks().installed() || stream_hooks().alloc_words(4 * kPairs, &h, &d) != 0) return false;
            for (unsigned long long i = 0; i < kPairs; ++i)
                free_.push_back(Pair{reinterpret_cast<std::atomic<unsigned long long>*>(h) + 4 * i, static_cast<char*>(d) + 32 * i});
        }
        out = free_.back();
        free_.pop_back();
        return true;
    }
    void release(const Pair& p)
    {
        std::lock_guard<std::mutex> g(mu_);
        free_.push_back(p);
    }

private:
    std::mutex        mu_;
    std::vector<Pair> free_;
};

// Process default of the stream-ordered wait's time limit.
inline unsigned long long default_stream_wait_ns()
{
    static const unsigned long long ns = [] {
        const char* raw = std::getenv("SLIME_STREAM_WAIT_MS");
        char*       end = nullptr;
        const double ms = raw ? std::strtod(raw, &end) : 0.0;
        return (raw && end && *end == 0 && ms > 0) ? static_cast<unsigned long long>(ms * 1e6) : 1000000000ull;
    }();
    return ns;
}

// DeviceSignal whose words the GPU can read and write: "ready" is set by a one-thread kernel in stream order
// (so the transfer engine posts only after the producer kernels on that stream have finished), "done" can be waited
// for by a bounded one-thread kernel in stream order (so consumer kernels queue behind the transfer without a host
// round trip). The reference does this with cuStreamWriteValue32 / cuStreamWaitValue32
// (dlslime/csrc/device/cuda/cuda_signal.h:40-118 in the reference); kernels give the wait a time limit, and a wait
// that runs into it sets the third word, which turns the operation's status into TIME_OUT (402): the stream went on
// without the data, and the caller must be told.
class MappedSignal final: public DeviceSignal {
public:
    explicit MappedSignal(const MappedWordPool::Pair& w): w_(w) { reset_all(); }
    ~MappedSignal() override { MappedWordPool::get().release(w_); }
    void init() override { reset_all(); }
    void record_gpu_ready() override
    {
        SLIME_NVTX_RANGE("slime.signal.record_gpu_ready", kNvtxSignal);
        if (stream_ != nullptr && stream_hooks().record_value(stream_, w_.dev, 1ull) == 0) return;
        w_.host[0].store(1, std::memory_order_release);
    }
    bool     is_gpu_ready() const override { return w_.host[0].load(std::memory_order_acquire) != 0; }
    uint32_t get_comm_done_mask() const override { return static_cast<uint32_t>(w_.host[1].load(std::memory_order_acquire)); }
    void     set_comm_done(int lane) override
    {
        w_.host[1].fetch_or(1ull << lane, std::memory_order_acq_rel);
        notify();
    }
    void bind_stream(void* stream) override { stream_ = stream; }
    void wait_comm_done_on_stream(uint32_t mask) override
    {
        SLIME_NVTX_RANGE("slime.signal.wait_comm_done_on_stream", kNvtxSignal);
        if (stream_ != nullptr)
            stream_hooks().wait_mask(stream_, static_cast<char*>(w_.dev) + 8, mask, limit_ns_ ? limit_ns_ : default_stream_wait_ns(),
                                     static_cast<char*>(w_.dev) + 16);
    }
    bool stream_wait_timed_out() const override { return w_.host[2].load(std::memory_order_acquire) != 0; }
    void set_stream_wait_limit_ns(unsigned long long ns) override { limit_ns_ = ns; }
    bool wait_comm_done_cpu(uint32_t mask, int64_t timeout_ms = -1) override
    {
        SLIME_NVTX_RANGE("slime.signal.wait_comm_done_cpu", kNvtxWait);
        auto satisfied = [&] { return forced_.load(std::memory_order_acquire) || (get_comm_done_mask() & mask) == mask; };
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
        // a kernel that waits for "done" in stream order must not be left to its time limit
        w_.host[1].store(~0ull, std::memory_order_release);
        notify();
    }
    void reset_all() override
    {
        w_.host[0].store(0, std::memory_order_relaxed);
        w_.host[1].store(0, std::memory_order_relaxed);
        w_.host[2].store(0, std::memory_order_relaxed);
        forced_.store(false, std::memory_order_release);
    }

private:
    void notify()
    {
        std::lock_guard<std::mutex> g(mu_);
        cv_.notify_all();
    }
    MappedWordPool::Pair    w_;
    unsigned long long      limit_ns_ = 0;
    std::atomic<bool>       forced_{false};
    void*                   stream_ = nullptr;
    std::mutex              mu_;
    std::condition_variable cv_;
};

// bypass = true: host-only signal (buffers are taken to be ready when the call is made). bypass = false: a
// stream-ordered signal when a CUDA layer installed its hooks, else the host-only one.
inline std::shared_ptr<DeviceSignal> create_signal(bool bypass = true)
{
    if (!bypass && stream_hooks().installed()) {
        MappedWordPool::Pair w;
        if (MappedWordPool::get().acquire(w)) return std::make_shared<MappedSignal>(w);
    }
    auto s = std::make_shared<HostSignal>();
    s->init();
    return s;
}

}  // namespace slime
