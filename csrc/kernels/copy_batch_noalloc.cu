// Batched segment copy whose scratch (segment table + counters) is a fixed device array
// inside the library image, so the call path never touches an allocator. See
// slime_noalloc.h for who needs this and for the rules of use. The copy loop is the same
// scheme as the endpoint's batched transfer: 64 KiB units over all segments, persistent
// CTAs, 16-byte vectors with eight loads in flight per thread, bytes for ragged edges.
#include <mutex>

#include "common/host_utils.h"
#include "slime_cuda.h"
#include "slime_noalloc.h"

using namespace slime;

namespace {

constexpr unsigned long long kUnit    = 64ull << 10;
constexpr int                kThreads = 256;
constexpr int                kMaxDev  = 64;

struct Seg {
    unsigned long long dst, src, len, first_unit;
};
static_assert(sizeof(Seg) == 32, "table entries are 32 bytes");

// [0, 256): reserved for counters of later variants (this variant needs none, so nothing has to start at zero)
// [256, ...): segment table, rewritten in full by every call before its kernel runs
static __device__ __align__(256) unsigned char g_scratch[SLIME_NOALLOC_SCRATCH_BYTES];

__device__ __forceinline__ void copy_bytes(unsigned char* dst, const unsigned char* src, unsigned long long n)
{
    const unsigned long long a = reinterpret_cast<unsigned long long>(dst), b = reinterpret_cast<unsigned long long>(src);
    if (((a | b) & 15) == 0) {
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
        for (unsigned long long k = (nv << 4) + threadIdx.x; k < n; k += kThreads) dst[k] = src[k];
    }
    else {
        for (unsigned long long k = threadIdx.x; k < n; k += kThreads) dst[k] = src[k];
    }
}

// `table` is the device address of g_scratch + 256, resolved on the host with cudaGetSymbolAddress.
__global__ void __launch_bounds__(kThreads) copy_batch_kernel(const Seg* __restrict__ table, int n_seg, unsigned long long n_units)
{
    __shared__ Seg s;
    for (unsigned long long u = blockIdx.x; u < n_units; u += gridDim.x) {
        if (threadIdx.x == 0) {
            int lo = 0, hi = n_seg - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (table[mid].first_unit <= u)
                    lo = mid;
                else
                    hi = mid - 1;
            }
            s = table[lo];
        }
        __syncthreads();
        const unsigned long long off = (u - s.first_unit) * kUnit;
        const unsigned long long n   = min(kUnit, s.len - off);
        copy_bytes(reinterpret_cast<unsigned char*>(s.dst + off), reinterpret_cast<const unsigned char*>(s.src + off), n);
        __syncthreads();
    }
}

// Per-device address of the scratch array. The array's name is only a host-side stand-in in host
// code; what a kernel needs is the address this query returns, with that device current.
unsigned char* g_scratch_addr[kMaxDev] = {nullptr};
std::mutex     g_setup_mu;

int scratch_for_current_device(unsigned char** out)
{
    int dev = 0;
    SLIME_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDev) return fail("no-alloc copy: device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> g(g_setup_mu);
    if (g_scratch_addr[dev] == nullptr) {
        void*       p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_scratch);
        if (e != cudaSuccess) return fail("no-alloc copy: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_scratch_addr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace

extern "C" {

int slime_copy_batch_noalloc_max_segments(void)
{
    return SLIME_NOALLOC_MAX_SEGMENTS;
}

int slime_copy_batch_noalloc(const unsigned long long* dst, const unsigned long long* src, const unsigned long long* len,
                             int n, void* stream_v)
{
    if (n < 0) return fail("no-alloc copy: negative segment count");
    if (n > SLIME_NOALLOC_MAX_SEGMENTS)
        return fail("no-alloc copy: %d segments exceed the fixed table of %d; split the batch", n, SLIME_NOALLOC_MAX_SEGMENTS);
    if (n == 0) return 0;
    if (dst == nullptr || src == nullptr || len == nullptr) return fail("no-alloc copy: null argument array");
    cudaStream_t   stream  = static_cast<cudaStream_t>(stream_v);
    // The table below is copied from this function's stack at call time; a capturing stream would record the
    // copy for later instead, when the stack is gone.
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    SLIME_CUDA_OK(cudaStreamIsCapturing(stream, &capturing));
    if (capturing != cudaStreamCaptureStatusNone)
        return fail("no-alloc copy: the stream is being captured; this call reads its arguments when it is made");
    unsigned char* scratch = nullptr;
    if (scratch_for_current_device(&scratch)) return -1;

    // Build the table on the stack in pieces and copy each piece into the device array. The pieces are
    // pageable host memory, so each copy has consumed its source when cudaMemcpyAsync returns.
    constexpr int      kPiece = 128;
    Seg                piece[kPiece];
    unsigned long long units = 0;
    Seg*               table = reinterpret_cast<Seg*>(scratch + 256);
    for (int base = 0; base < n; base += kPiece) {
        const int m = n - base < kPiece ? n - base : kPiece;
        for (int i = 0; i < m; ++i) {
            Seg& s       = piece[i];
            s.dst        = dst[base + i];
            s.src        = src[base + i];
            s.len        = len[base + i];
            s.first_unit = units;
            if (s.len != 0 && (s.dst == 0 || s.src == 0)) return fail("no-alloc copy: segment %d has a null address", base + i);
            units += (s.len + kUnit - 1) / kUnit;
        }
        SLIME_CUDA_OK(cudaMemcpyAsync(table + base, piece, sizeof(Seg) * m, cudaMemcpyHostToDevice, stream));
    }
    if (units == 0) return 0;
    const unsigned long long cap  = static_cast<unsigned long long>(sm_count()) * 8;
    const int                grid = static_cast<int>(units < cap ? units : cap);
    copy_batch_kernel<<<grid, kThreads, 0, stream>>>(table, n, units);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

}  // extern "C"
