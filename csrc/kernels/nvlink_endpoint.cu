// NVLink endpoint: memory-region registry over CUDA IPC plus ONE kernel that moves
// a whole batch of (local offset, remote offset, length) segments between this
// GPU and peer GPUs. Counterpart of the reference's NVLinkEndpoint / NVLinkMemoryPool
// (dlslime/csrc/engine/nvlink/nvlink_endpoint.h:22-47, memory_pool.cpp:19-153 in the
// reference), which issues one cudaMemcpyAsync per segment and can only read. Here a
// batch is one launch, both directions exist, and a completion word (local, remote
// or mapped host memory) can be published when the last byte has landed, which is
// what write_with_imm / imm_recv are built from.
//
// Work is cut into 64 KiB units over all segments; persistent CTAs walk the units.
// Aligned units move as 16-byte vectors with eight loads in flight per thread;
// ragged heads and tails fall back to bytes.
#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include <cstdlib>

#include "common/host_utils.h"
#include "common/ptx.cuh"
#include "slime_cuda.h"

using namespace slime;

namespace {

constexpr unsigned long long kUnitBytes  = 64ull << 10;
constexpr int                kInlineSegs = 8;
constexpr int                kThreads    = 256;

struct Segment {
    unsigned long long dst;
    unsigned long long src;
    unsigned long long len;
    unsigned long long first_unit;  // index of this segment's first unit in the batch
};

struct InlineBatch {
    Segment seg[kInlineSegs];
};

struct CopyArgs {
    const Segment*      table;  // device table, or nullptr when `inl` is used
    int                 n_seg;
    unsigned long long  n_units;
    unsigned long long* signal;  // optional completion word
    unsigned long long  signal_value;
    int                 signal_add;
    unsigned int*       block_counter;
    unsigned long long  unit_bytes;  // work unit: kUnitBytes, or smaller so that several CTAs share one piece
    KernelStatus*       status;      // where a wait that ran out is recorded (mapped host memory; may be null)
};

__device__ __forceinline__ void copy_unit(unsigned char* dst, const unsigned char* src, unsigned long long n)
{
    const unsigned long long mis = (reinterpret_cast<unsigned long long>(dst) | reinterpret_cast<unsigned long long>(src)) & 15;
    if (mis == 0) {
        const unsigned long long nv = n >> 4;
        const uint4*             s  = reinterpret_cast<const uint4*>(src);
        uint4*                   d  = reinterpret_cast<uint4*>(dst);
        unsigned long long       i  = threadIdx.x;
        for (; i + 7ull * kThreads < nv; i += 8ull * kThreads) {
            uint4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = s[i + j * kThreads];
#pragma unroll
            for (int j = 0; j < 8; ++j) d[i + j * kThreads] = v[j];
        }
        for (; i < nv; i += kThreads) d[i] = s[i];
        for (unsigned long long b = (nv << 4) + threadIdx.x; b < n; b += kThreads) dst[b] = src[b];
    }
    else if (((reinterpret_cast<unsigned long long>(dst) ^ reinterpret_cast<unsigned long long>(src)) & 15) == 0) {
        // same misalignment on both sides: byte head, vector body, byte tail
        unsigned long long head = 16 - (reinterpret_cast<unsigned long long>(dst) & 15);
        if (head > n) head = n;
        for (unsigned long long b = threadIdx.x; b < head; b += kThreads) dst[b] = src[b];
        const unsigned long long nv = (n - head) >> 4;
        const uint4*             s  = reinterpret_cast<const uint4*>(src + head);
        uint4*                   d  = reinterpret_cast<uint4*>(dst + head);
        for (unsigned long long i = threadIdx.x; i < nv; i += kThreads) d[i] = s[i];
        for (unsigned long long b = head + (nv << 4) + threadIdx.x; b < n; b += kThreads) dst[b] = src[b];
    }
    else {
        for (unsigned long long b = threadIdx.x; b < n; b += kThreads) dst[b] = src[b];
    }
}

__global__ void __launch_bounds__(kThreads) p2p_scatter_gather_kernel(CopyArgs a, InlineBatch inl)
{
    __shared__ Segment s_seg;
    for (unsigned long long u = blockIdx.x; u < a.n_units; u += gridDim.x) {
        if (threadIdx.x == 0) {
            // binary search for the segment that owns unit u
            int lo = 0, hi = a.n_seg - 1;
            while (lo < hi) {
                const int                mid = (lo + hi + 1) >> 1;
                const unsigned long long fu  = a.table ? a.table[mid].first_unit : inl.seg[mid].first_unit;
                if (fu <= u)
                    lo = mid;
                else
                    hi = mid - 1;
            }
            s_seg = a.table ? a.table[lo] : inl.seg[lo];
        }
        __syncthreads();
        const unsigned long long off = (u - s_seg.first_unit) * a.unit_bytes;
        const unsigned long long n   = min(a.unit_bytes, s_seg.len - off);
        copy_unit(reinterpret_cast<unsigned char*>(s_seg.dst + off), reinterpret_cast<const unsigned char*>(s_seg.src + off), n);
        __syncthreads();
    }
    if (a.signal != nullptr) {
        __shared__ bool is_last;
        __syncthreads();
        if (threadIdx.x == 0) {
            fence_acq_rel_sys();
            is_last = atomicAdd(a.block_counter, 1u) == gridDim.x - 1;
            if (is_last) {
                fence_acq_rel_sys();
                if (a.signal_add)
                    red_add_release_sys(a.signal, a.signal_value);
                else
                    st_release_sys(a.signal, a.signal_value);
                *a.block_counter = 0;
            }
        }
    }
}

// The same batch through the bulk-copy engine, for batches whose addresses and lengths are all multiples of 16 bytes.
// One thread per CTA drives a ring of shared-memory buffers over the CTA's whole sequence of 8 KiB chunks (unit after
// unit, with no drain between units): global -> shared bulk loads (peer memory included) run ahead of the shared ->
// global bulk stores by the ring depth, and a buffer is reloaded as soon as the copy engine has read it. What the
// engine buys over the 256-thread load/store kernel is occupancy: one warp per CTA instead of eight, so a transfer
// that runs beside compute kernels takes almost no issue slots from them.
//
// A wait that runs out is recorded in the status page, the CTA stops issuing, and the batch's completion word is NOT
// published (by any CTA: the last one to report in looks at the status page first), so a future on it times out
// instead of reporting bytes that never landed.
constexpr int kBulkBufs  = 8;
constexpr int kBulkChunk = 8192;
constexpr int kBulkLag   = 2;  // stores that may still be reading their buffers when the next load is issued

struct BulkCursor {
    unsigned long long unit;   // current unit (blockIdx.x, + gridDim.x, ...)
    unsigned long long src, dst, bytes;  // of the unit
    unsigned long long done;   // bytes of the unit already consumed by this cursor
    bool               valid;
};

__device__ __forceinline__ void bulk_cursor_load_unit(const CopyArgs& a, const InlineBatch& inl, BulkCursor& c)
{
    c.valid = c.unit < a.n_units;
    if (!c.valid) return;
    int lo = 0, hi = a.n_seg - 1;
    while (lo < hi) {
        const int                mid = (lo + hi + 1) >> 1;
        const unsigned long long fu  = a.table ? a.table[mid].first_unit : inl.seg[mid].first_unit;
        if (fu <= c.unit)
            lo = mid;
        else
            hi = mid - 1;
    }
    const Segment            seg = a.table ? a.table[lo] : inl.seg[lo];
    const unsigned long long off = (c.unit - seg.first_unit) * a.unit_bytes;
    c.src   = seg.src + off;
    c.dst   = seg.dst + off;
    c.bytes = min(a.unit_bytes, seg.len - off);
    c.done  = 0;
}

// Returns the size of the cursor's next chunk and its addresses, and advances the cursor.
__device__ __forceinline__ uint32_t bulk_cursor_next(const CopyArgs& a, const InlineBatch& inl, BulkCursor& c,
                                                     unsigned long long* src, unsigned long long* dst)
{
    const uint32_t n = static_cast<uint32_t>(min(static_cast<unsigned long long>(kBulkChunk), c.bytes - c.done));
    *src = c.src + c.done;
    *dst = c.dst + c.done;
    c.done += n;
    if (c.done >= c.bytes) {
        c.unit += gridDim.x;
        bulk_cursor_load_unit(a, inl, c);
    }
    return n;
}

__global__ void __launch_bounds__(32) p2p_bulk_kernel(CopyArgs a, InlineBatch inl)
{
    extern __shared__ __align__(128) unsigned char bulk_smem[];
    __shared__ uint64_t bars[kBulkBufs];
    if (threadIdx.x == 0) {
        for (int b = 0; b < kBulkBufs; ++b) mbar_init(&bars[b], 1);
        fence_mbar_init();
        BulkCursor ld{}, st{};
        ld.unit = st.unit = blockIdx.x;
        bulk_cursor_load_unit(a, inl, ld);
        bulk_cursor_load_unit(a, inl, st);
        unsigned long long n_ld = 0, n_st = 0;
        auto issue_load = [&]() {
            const int          b = static_cast<int>(n_ld % kBulkBufs);
            unsigned long long src, dst;
            const uint32_t     bytes = bulk_cursor_next(a, inl, ld, &src, &dst);
            mbar_arrive_expect_tx(&bars[b], bytes);
            bulk_load_g2s(bulk_smem + b * kBulkChunk, reinterpret_cast<const void*>(src), bytes, &bars[b]);
            ++n_ld;
        };
        while (n_ld < kBulkBufs - kBulkLag && ld.valid) issue_load();
        bool ok = true;
        while (st.valid) {
            const int b = static_cast<int>(n_st % kBulkBufs);
            if (!mbar_wait(&bars[b], static_cast<uint32_t>((n_st / kBulkBufs) & 1), a.status, 20, b)) {
                ok = false;  // the load never landed: stop issuing, leave through the common exit
                break;
            }
            unsigned long long src, dst;
            const uint32_t     bytes = bulk_cursor_next(a, inl, st, &src, &dst);
            bulk_store_s2g(reinterpret_cast<void*>(dst), bulk_smem + b * kBulkChunk, bytes);
            tma_store_commit();
            ++n_st;
            if (ld.valid) {
                // the buffer the next load goes into was read by store number n_ld - kBulkBufs, which is at least
                // kBulkLag stores back: wait until only the most recent kBulkLag stores may still be reading
                tma_store_wait_read<kBulkLag>();
                issue_load();
            }
        }
        tma_store_wait<0>();  // every byte has been written before the CTA reports in
        fence_proxy_async();
        (void)ok;
        if (a.signal != nullptr) {
            fence_acq_rel_sys();
            if (atomicAdd(a.block_counter, 1u) == gridDim.x - 1) {
                fence_acq_rel_sys();
                // a CTA whose wait ran out has recorded it before counting itself in
                const bool failed = a.status != nullptr && *reinterpret_cast<volatile unsigned int*>(&a.status->code) != 0;
                if (!failed) {
                    if (a.signal_add)
                        red_add_release_sys(a.signal, a.signal_value);
                    else
                        st_release_sys(a.signal, a.signal_value);
                }
                *a.block_counter = 0;
            }
        }
    }
}

struct Region {
    std::string        name;
    unsigned long long addr   = 0;  // usable address in this process (already includes offset)
    unsigned long long offset = 0;  // offset of addr inside its allocation (exported with the handle)
    unsigned long long length = 0;
    unsigned char      ipc[64];
    void*              mapped_base = nullptr;  // remote only: what cudaIpcOpenMemHandle returned
    bool               alive       = false;
};

struct StagingSlot {
    Segment*    host = nullptr;
    Segment*    dev  = nullptr;
    cudaEvent_t done = nullptr;
};

constexpr int kStagingSlots   = 8;
constexpr int kStagingEntries = 1 << 16;

struct Endpoint {
    std::mutex                 mu;
    std::vector<Region>        local, remote;
    std::map<std::string, int> local_by_name, remote_by_name;
    std::map<std::string, void*> opened;  // ipc handle bytes -> mapped base (one open per allocation)
    StagingSlot                slots[kStagingSlots];
    int                        next_slot = 0;
    unsigned int*              counters  = nullptr;  // one block counter per staging slot
    int                        next_counter = 0;
    int                        device = 0;
    KernelStatus*              status_host = nullptr;  // mapped page the bulk kernel reports into
    KernelStatus*              status_dev  = nullptr;
    std::mutex                 submit_mu;  // the staging-slot and counter cursors, when threads share an endpoint
};

int ensure_staging(Endpoint* ep)
{
    if (ep->counters) return 0;
    SLIME_CUDA_OK(cudaGetDevice(&ep->device));
    SLIME_CUDA_OK(cudaMalloc(&ep->counters, sizeof(unsigned int) * 64));
    SLIME_CUDA_OK(cudaMemset(ep->counters, 0, sizeof(unsigned int) * 64));
    void *sh = nullptr, *sd = nullptr;
    if (slime_status_alloc(&sh, &sd)) return -1;
    ep->status_host = static_cast<KernelStatus*>(sh);
    ep->status_dev  = static_cast<KernelStatus*>(sd);
    return 0;
}

// Work unit of the batched kernels. 64 KiB by default; SLIME_NVLINK_UNIT_KB (16 .. 1024, a multiple of 16) overrides
// it, e.g. 16 so that four CTAs work on each 64 KiB piece at the same time.
std::atomic<unsigned long long> g_unit_bytes{0};  // 0 = not decided yet
std::atomic<int>                g_bulk{-1};       // -1 = not decided yet

unsigned long long unit_bytes_setting()
{
    unsigned long long v = g_unit_bytes.load(std::memory_order_relaxed);
    if (v == 0) {
        const char* raw = std::getenv("SLIME_NVLINK_UNIT_KB");
        const long  kb  = raw ? std::strtol(raw, nullptr, 10) : 0;
        v = (kb >= 16 && kb <= 1024 && kb % 16 == 0) ? static_cast<unsigned long long>(kb) << 10 : kUnitBytes;
        g_unit_bytes.store(v, std::memory_order_relaxed);
    }
    return v;
}

bool bulk_setting()
{
    int v = g_bulk.load(std::memory_order_relaxed);
    if (v < 0) {
        v = std::getenv("SLIME_NVLINK_NO_BULK") == nullptr ? 1 : 0;
        g_bulk.store(v, std::memory_order_relaxed);
    }
    return v != 0;
}

// All staging slots are set up by the first batch that needs a table: one pinned block and one device block cut into
// kStagingSlots tables. (Allocating slot by slot put a cudaHostAlloc and a cudaMalloc, both synchronous and
// milliseconds long, into each of the first kStagingSlots large batches of an endpoint.)
int ensure_slots(Endpoint* ep)
{
    if (ep->slots[0].host) return 0;
    Segment *host = nullptr, *dev = nullptr;
    SLIME_CUDA_OK(cudaHostAlloc(reinterpret_cast<void**>(&host), sizeof(Segment) * kStagingEntries * kStagingSlots, cudaHostAllocPortable));
    SLIME_CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&dev), sizeof(Segment) * kStagingEntries * kStagingSlots));
    for (int i = 0; i < kStagingSlots; ++i) {
        ep->slots[i].host = host + static_cast<size_t>(i) * kStagingEntries;
        ep->slots[i].dev  = dev + static_cast<size_t>(i) * kStagingEntries;
        SLIME_CUDA_OK(cudaEventCreateWithFlags(&ep->slots[i].done, cudaEventDisableTiming));
    }
    return 0;
}

}  // namespace

extern "C" {

void* slime_nvlink_ep_create(void)
{
    return new Endpoint();
}

int slime_nvlink_ep_destroy(void* h)
{
    Endpoint* ep = static_cast<Endpoint*>(h);
    if (!ep) return 0;
    for (auto& kv : ep->opened) cudaIpcCloseMemHandle(kv.second);
    if (ep->slots[0].host) cudaFreeHost(ep->slots[0].host);  // one block each for all slots
    if (ep->slots[0].dev) cudaFree(ep->slots[0].dev);
    for (auto& s : ep->slots)
        if (s.done) cudaEventDestroy(s.done);
    if (ep->counters) cudaFree(ep->counters);
    if (ep->status_host) slime_status_free(ep->status_host);
    delete ep;
    return 0;
}

// Registers [addr, addr+length) as a local region. The IPC handle of the enclosing
// allocation and the offset of addr inside it are recorded for export.
// Returns the handle (>= 0). Registering the same name again replaces the entry.
int slime_nvlink_ep_register(void* h, unsigned long long addr, unsigned long long length, const char* name)
{
    Endpoint* ep = static_cast<Endpoint*>(h);
    Region    r;
    r.addr   = addr;
    r.length = length;
    r.alive  = true;
    unsigned long long off = 0;
    if (slime_ipc_get_handle(reinterpret_cast<const void*>(addr), r.ipc, &off, nullptr)) {
        // Memory that CUDA IPC cannot export (for example virtual-memory-managed pools) can still be
        // used by endpoints of the same process; other processes will fail to open the zero handle.
        memset(r.ipc, 0, 64);
        off = 0;
        cudaGetLastError();
    }
    r.offset = off;
    std::lock_guard<std::mutex> g(ep->mu);
    char                        auto_name[64];
    if (name == nullptr || name[0] == 0) {
        snprintf(auto_name, sizeof(auto_name), "auto_0x%llx", addr);
        name = auto_name;
    }
    r.name  = name;
    auto it = ep->local_by_name.find(r.name);
    if (it != ep->local_by_name.end()) {
        ep->local[it->second] = r;
        return it->second;
    }
    ep->local.push_back(r);
    ep->local_by_name[r.name] = static_cast<int>(ep->local.size()) - 1;
    return static_cast<int>(ep->local.size()) - 1;
}

int slime_nvlink_ep_unregister(void* h, int handle)
{
    Endpoint*                   ep = static_cast<Endpoint*>(h);
    std::lock_guard<std::mutex> g(ep->mu);
    if (handle < 0 || handle >= static_cast<int>(ep->local.size()) || !ep->local[handle].alive)
        return fail("nvlink endpoint: no local region with handle %d", handle);
    ep->local_by_name.erase(ep->local[handle].name);
    ep->local[handle].alive = false;
    return 0;
}

// Fills `out` (64 bytes handle, then offset, addr, length as u64) for local handle.
int slime_nvlink_ep_local_info(void* h, int handle, unsigned char* ipc_out64, unsigned long long* offset,
                               unsigned long long* addr, unsigned long long* length)
{
    Endpoint*                   ep = static_cast<Endpoint*>(h);
    std::lock_guard<std::mutex> g(ep->mu);
    if (handle < 0 || handle >= static_cast<int>(ep->local.size()) || !ep->local[handle].alive)
        return fail("nvlink endpoint: no local region with handle %d", handle);
    const Region& r = ep->local[handle];
    memcpy(ipc_out64, r.ipc, 64);
    *offset = r.offset;
    *addr   = r.addr;
    *length = r.length;
    return 0;
}

// Maps a peer's region. same_process != 0 means `addr` is directly usable (both
// endpoints live in one process, where an IPC handle cannot be opened).
int slime_nvlink_ep_register_remote(void* h, const char* name, const unsigned char* ipc64, unsigned long long offset,
                                    unsigned long long length, unsigned long long addr, int same_process)
{
    Endpoint* ep = static_cast<Endpoint*>(h);
    Region    r;
    r.name   = name ? name : "";
    r.offset = offset;
    r.length = length;
    r.alive  = true;
    memcpy(r.ipc, ipc64, 64);
    std::lock_guard<std::mutex> g(ep->mu);
    if (same_process) {
        r.addr = addr;
    }
    else {
        const std::string key(reinterpret_cast<const char*>(ipc64), 64);
        auto              it = ep->opened.find(key);
        void*             base = nullptr;
        if (it == ep->opened.end()) {
            if (slime_ipc_open(ipc64, &base)) return -1;
            ep->opened[key] = base;
        }
        else {
            base = it->second;
        }
        r.mapped_base = base;
        r.addr        = reinterpret_cast<unsigned long long>(base) + offset;
    }
    auto it = ep->remote_by_name.find(r.name);
    if (!r.name.empty() && it != ep->remote_by_name.end()) {
        ep->remote[it->second] = r;
        return it->second;
    }
    ep->remote.push_back(r);
    if (!r.name.empty()) ep->remote_by_name[r.name] = static_cast<int>(ep->remote.size()) - 1;
    return static_cast<int>(ep->remote.size()) - 1;
}

int slime_nvlink_ep_handle(void* h, const char* name, int remote)
{
    Endpoint*                   ep = static_cast<Endpoint*>(h);
    std::lock_guard<std::mutex> g(ep->mu);
    auto&                       m  = remote ? ep->remote_by_name : ep->local_by_name;
    auto                        it = m.find(name);
    return it == m.end() ? -1 : it->second;
}

unsigned long long slime_nvlink_ep_remote_addr(void* h, int handle)
{
    Endpoint*                   ep = static_cast<Endpoint*>(h);
    std::lock_guard<std::mutex> g(ep->mu);
    if (handle < 0 || handle >= static_cast<int>(ep->remote.size())) return 0;
    return ep->remote[handle].addr;
}

// Status page of the endpoint's kernels: code (0 = ok, 402 = a copy never landed), site, block and aux word.
// Returns 0 and zeros when no kernel of this endpoint has run yet.
int slime_nvlink_ep_status(void* h, unsigned int* out4)
{
    Endpoint* ep = static_cast<Endpoint*>(h);
    out4[0] = out4[1] = out4[2] = out4[3] = 0;
    if (ep == nullptr || ep->status_host == nullptr) return 0;
    const volatile KernelStatus* st = ep->status_host;
    out4[0] = st->code;
    out4[1] = st->where;
    out4[2] = st->block;
    out4[3] = st->aux;
    return 0;
}

int slime_nvlink_ep_status_clear(void* h)
{
    Endpoint* ep = static_cast<Endpoint*>(h);
    if (ep != nullptr && ep->status_host != nullptr) memset(ep->status_host, 0, sizeof(KernelStatus));
    return 0;
}

// Tuning of the batched kernels for the whole process: unit_kb (16 .. 1024, a multiple of 16; 0 = leave) is the work
// unit CTAs take from a batch, bulk (0 / 1; negative = leave) picks between the 256-thread load/store kernel and the
// bulk-copy-engine kernel for batches that are 16-byte aligned throughout. The same as SLIME_NVLINK_UNIT_KB and
// SLIME_NVLINK_NO_BULK, but changeable between calls (benchmarks sweep it).
int slime_nvlink_ep_tune(int unit_kb, int bulk)
{
    if (unit_kb != 0) {
        if (unit_kb < 16 || unit_kb > 1024 || unit_kb % 16 != 0) return fail("nvlink endpoint: unit of %d KiB not in [16, 1024] or not a multiple of 16", unit_kb);
        g_unit_bytes.store(static_cast<unsigned long long>(unit_kb) << 10);
    }
    if (bulk >= 0) g_bulk.store(bulk ? 1 : 0);
    return 0;
}

// Few, large pieces are a job for the copy engines: no SM is occupied, nothing is staged, and for one contiguous
// region a DMA copy is a few percent faster than any kernel (it has no tail and no launch-shaped ramp). The kernels
// take over where the copy engines lose: many pieces, each of which would cost one host call and one DMA set-up.
constexpr int                kCopyEngineMaxSegs  = 4;
constexpr unsigned long long kCopyEngineMinBytes = 4ull << 20;

static bool copy_engine_enabled()
{
    static const bool off = std::getenv("SLIME_NVLINK_NO_COPY_ENGINE") != nullptr;
    return !off;
}

// Checks one assignment against its regions and resolves it to device addresses (ep->mu held by the caller).
static int resolve_segment(Endpoint* ep, int index, long long lh, long long rh, unsigned long long roff,
                           unsigned long long loff, unsigned long long len, int is_write, unsigned long long* dst,
                           unsigned long long* src)
{
    if (lh < 0 || lh >= static_cast<long long>(ep->local.size()) || !ep->local[lh].alive)
        return fail("nvlink endpoint: assignment %d names unknown local region %lld", index, lh);
    if (rh < 0 || rh >= static_cast<long long>(ep->remote.size()) || !ep->remote[rh].alive)
        return fail("nvlink endpoint: assignment %d names unknown remote region %lld", index, rh);
    const Region& L = ep->local[lh];
    const Region& R = ep->remote[rh];
    // written so that no sum can wrap: an offset near 2^64 (a negative number on the caller's side) is refused
    if (loff > L.length || len > L.length - loff || roff > R.length || len > R.length - roff)
        return fail("nvlink endpoint: assignment %d exceeds a region (local %llu+%llu of %llu, remote %llu+%llu of %llu)", index,
                    loff, len, L.length, roff, len, R.length);
    *dst = is_write ? R.addr + roff : L.addr + loff;
    *src = is_write ? L.addr + loff : R.addr + roff;
    return 0;
}

// One contiguous piece, arguments as scalars (no table to build on the caller's side): a DMA copy in stream order,
// followed by the completion word if one is asked for.
int slime_nvlink_ep_copy1(void* h, long long local_handle, long long remote_handle, unsigned long long remote_offset,
                          unsigned long long local_offset, unsigned long long length, int is_write, void* signal,
                          unsigned long long signal_value, void* stream_v)
{
    Endpoint*          ep     = static_cast<Endpoint*>(h);
    cudaStream_t       stream = static_cast<cudaStream_t>(stream_v);
    unsigned long long dst = 0, src = 0;
    {
        std::lock_guard<std::mutex> g(ep->mu);
        if (resolve_segment(ep, 0, local_handle, remote_handle, remote_offset, local_offset, length, is_write, &dst, &src))
            return -1;
    }
    if (length)
        SLIME_CUDA_OK(cudaMemcpyAsync(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), length,
                                      cudaMemcpyDeviceToDevice, stream));
    if (signal) return slime_signal_flag_kernel(signal, signal_value, 0, stream_v);
    return 0;
}

// One batched transfer. tuples = n x {local_handle, remote_handle, remote_offset, local_offset, length}
// (the assignment tuple order of the endpoint API). is_write: local -> remote, else remote -> local.
// signal (optional) receives signal_value (store, or add when signal_add) after the last byte.
int slime_nvlink_ep_transfer(void* h, const unsigned long long* tuples, int n, int is_write, void* signal,
                             unsigned long long signal_value, int signal_add, int max_blocks, void* stream_v)
{
    Endpoint*    ep     = static_cast<Endpoint*>(h);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (n < 0) return fail("nvlink endpoint: negative batch size");
    if (n == 0 && signal == nullptr) return 0;
    if (n >= 1 && n <= kCopyEngineMaxSegs && copy_engine_enabled()) {
        bool large = true;
        for (int i = 0; i < n; ++i) large = large && (n == 1 || tuples[5ull * i + 4] >= kCopyEngineMinBytes);
        if (large) {
            unsigned long long dst[kCopyEngineMaxSegs], src[kCopyEngineMaxSegs];
            {
                std::lock_guard<std::mutex> g(ep->mu);
                for (int i = 0; i < n; ++i) {
                    const unsigned long long* t = tuples + 5ull * i;
                    if (resolve_segment(ep, i, static_cast<long long>(t[0]), static_cast<long long>(t[1]), t[2], t[3], t[4],
                                        is_write, &dst[i], &src[i]))
                        return -1;
                }
            }
            for (int i = 0; i < n; ++i)
                if (tuples[5ull * i + 4])
                    SLIME_CUDA_OK(cudaMemcpyAsync(reinterpret_cast<void*>(dst[i]), reinterpret_cast<const void*>(src[i]),
                                                  tuples[5ull * i + 4], cudaMemcpyDeviceToDevice, stream));
            if (signal) return slime_signal_flag_kernel(signal, signal_value, signal_add, stream_v);
            return 0;
        }
    }
    std::lock_guard<std::mutex> submit(ep->submit_mu);
    if (ensure_staging(ep)) return -1;
    const unsigned long long unit = unit_bytes_setting();
    int done = 0;
    do {
        const int          batch = std::min(n - done, kStagingEntries);
        InlineBatch        inl{};
        Segment*           seg_out = nullptr;
        StagingSlot*       slot    = nullptr;
        if (batch <= kInlineSegs) {
            seg_out = inl.seg;
        }
        else {
            if (ensure_slots(ep)) return -1;
            slot = &ep->slots[ep->next_slot];
            ep->next_slot = (ep->next_slot + 1) % kStagingSlots;
            SLIME_CUDA_OK(cudaEventSynchronize(slot->done));  // previous user of this slot has been consumed
            seg_out = slot->host;
        }
        unsigned long long units = 0;
        bool               all_aligned = true;
        {
            std::lock_guard<std::mutex> g(ep->mu);
            for (int i = 0; i < batch; ++i) {
                const unsigned long long* t  = tuples + 5ull * (done + i);
                const unsigned long long  len = t[4];
                Segment&                  s   = seg_out[i];
                if (resolve_segment(ep, done + i, static_cast<long long>(t[0]), static_cast<long long>(t[1]), t[2], t[3], len,
                                    is_write, &s.dst, &s.src))
                    return -1;
                s.len = len;
                if (((s.dst | s.src | len) & 15ull) != 0) all_aligned = false;
            }
        }
        for (int i = 0; i < batch; ++i) {
            seg_out[i].first_unit = units;
            units += (seg_out[i].len + unit - 1) / unit;
        }
        CopyArgs a{};
        a.n_seg      = batch;
        a.n_units    = units;
        a.unit_bytes = unit;
        a.status     = ep->status_dev;
        const bool last_batch = done + batch >= n;
        if (last_batch && signal != nullptr) {
            a.signal        = static_cast<unsigned long long*>(signal);
            a.signal_value  = signal_value;
            a.signal_add    = signal_add;
            a.block_counter = ep->counters + ep->next_counter;
            ep->next_counter = (ep->next_counter + 1) % 64;
        }
        if (slot) {
            SLIME_CUDA_OK(cudaMemcpyAsync(slot->dev, slot->host, sizeof(Segment) * batch, cudaMemcpyHostToDevice, stream));
            a.table = slot->dev;
        }
        if (all_aligned && bulk_setting() && units > 0) {
            // three 64 KiB rings fit in one SM's shared memory
            constexpr int kBulkSmem = kBulkBufs * kBulkChunk;
            static bool   configured[64] = {false};  // the attribute belongs to the device's copy of the function
            const int     dev_slot = ep->device >= 0 && ep->device < 64 ? ep->device : 0;
            if (!configured[dev_slot]) {
                SLIME_CUDA_OK(cudaFuncSetAttribute(p2p_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmem));
                SLIME_CUDA_OK(cudaFuncSetAttribute(p2p_bulk_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                                   cudaSharedmemCarveoutMaxShared));  // see prefer_max_shared_carveout
                configured[dev_slot] = true;
            }
            long long grid = static_cast<long long>(std::min<unsigned long long>(units, static_cast<unsigned long long>(sm_count()) * 3));
            if (max_blocks > 0 && grid > max_blocks) grid = max_blocks;
            p2p_bulk_kernel<<<static_cast<int>(grid), 32, kBulkSmem, stream>>>(a, inl);
        }
        else {
            long long grid = static_cast<long long>(std::min<unsigned long long>(units, static_cast<unsigned long long>(sm_count()) * 8));
            if (max_blocks > 0 && grid > max_blocks) grid = max_blocks;
            if (grid < 1) grid = 1;
            static bool carveout[64] = {false};  // transfers run beside compute kernels: see prefer_max_shared_carveout
            SLIME_CUDA_OK(prefer_max_shared_carveout(p2p_scatter_gather_kernel, carveout));
            p2p_scatter_gather_kernel<<<static_cast<int>(grid), kThreads, 0, stream>>>(a, inl);
        }
        SLIME_CUDA_OK(cudaGetLastError());
        if (slot) SLIME_CUDA_OK(cudaEventRecord(slot->done, stream));  // the slot is free once the kernel has read its table
        done += batch;
    } while (done < n);
    return 0;
}

}  // extern "C"
