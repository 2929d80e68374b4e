// Bounded lock-free multi-producer / multi-consumer ring of trivially copyable items
// (per-slot sequence numbers), plus a spin lock, a CPU pause hint and a monotonic clock.
// It plays the role of the reference's vendored jring (dlslime/csrc/common/jring.h in
// the reference): free-slot pools and the submit queues between user threads and the
// progress thread.
#pragma once

#include <atomic>
#include <chrono>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <new>
#include <stdexcept>

namespace slime {

inline void cpu_pause()
{
#if defined(__x86_64__) || defined(__i386__)
    __builtin_ia32_pause();
#elif defined(__aarch64__)
    asm volatile("yield" ::: "memory");
#endif
}

inline uint64_t monotonic_ns()
{
    return static_cast<uint64_t>(
        std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count());
}

class SpinLock {
public:
    void lock()
    {
        while (flag_.exchange(true, std::memory_order_acquire))
            while (flag_.load(std::memory_order_relaxed)) cpu_pause();
    }
    bool try_lock() { return !flag_.exchange(true, std::memory_order_acquire); }
    void unlock() { flag_.store(false, std::memory_order_release); }

private:
    std::atomic<bool> flag_{false};
};

template<typename T>
class MpmcRing {
public:
    explicit MpmcRing(size_t capacity_pow2): mask_(capacity_pow2 - 1), cells_(new Cell[capacity_pow2])
    {
        if (capacity_pow2 < 2 || (capacity_pow2 & mask_) != 0) throw std::invalid_argument("ring capacity must be a power of two >= 2");
        for (size_t i = 0; i <= mask_; ++i) cells_[i].seq.store(i, std::memory_order_relaxed);
    }

    bool try_push(const T& v)
    {
        size_t pos = tail_.load(std::memory_order_relaxed);
        for (;;) {
            Cell&    c   = cells_[pos & mask_];
            size_t   seq = c.seq.load(std::memory_order_acquire);
            intptr_t dif = static_cast<intptr_t>(seq) - static_cast<intptr_t>(pos);
            if (dif == 0) {
                if (tail_.compare_exchange_weak(pos, pos + 1, std::memory_order_relaxed)) {
                    c.value = v;
                    c.seq.store(pos + 1, std::memory_order_release);
                    return true;
                }
            }
            else if (dif < 0) {
                return false;  // full
            }
            else {
                pos = tail_.load(std::memory_order_relaxed);
            }
        }
    }

    bool try_pop(T& out)
    {
        size_t pos = head_.load(std::memory_order_relaxed);
        for (;;) {
            Cell&    c   = cells_[pos & mask_];
            size_t   seq = c.seq.load(std::memory_order_acquire);
            intptr_t dif = static_cast<intptr_t>(seq) - static_cast<intptr_t>(pos + 1);
            if (dif == 0) {
                if (head_.compare_exchange_weak(pos, pos + 1, std::memory_order_relaxed)) {
                    out = c.value;
                    c.seq.store(pos + mask_ + 1, std::memory_order_release);
                    return true;
                }
            }
            else if (dif < 0) {
                return false;  // empty
            }
            else {
                pos = head_.load(std::memory_order_relaxed);
            }
        }
    }

    // Pops up to n items; returns how many were taken.
    size_t pop_burst(T* out, size_t n)
    {
        size_t got = 0;
        while (got < n && try_pop(out[got])) ++got;
        return got;
    }

    void push_blocking(const T& v)
    {
        while (!try_push(v)) cpu_pause();
    }
    T pop_blocking()
    {
        T v;
        while (!try_pop(v)) cpu_pause();
        return v;
    }

    size_t capacity() const { return mask_ + 1; }
    size_t size_approx() const
    {
        size_t t = tail_.load(std::memory_order_relaxed), h = head_.load(std::memory_order_relaxed);
        return t >= h ? t - h : 0;
    }

private:
    struct alignas(64) Cell {
        std::atomic<size_t> seq;
        T                   value;
    };
    const size_t            mask_;
    std::unique_ptr<Cell[]> cells_;
    alignas(64) std::atomic<size_t> tail_{0};
    alignas(64) std::atomic<size_t> head_{0};
};

}  // namespace slime
