// CUDA-side plumbing that is not a hot kernel: error text, mapped status pages,
// host-visible flag words, the cudaMalloc + CUDA-IPC symmetric heap, and two
// one-thread kernels that wait on / publish a flag in stream order (the device
// replacement for stream memory operations, with a bounded wait).
#include "common/host_utils.h"
#include "common/ptx.cuh"
#include "slime_cuda.h"

using namespace slime;

namespace {

__global__ void wait_flag_kernel(const unsigned long long* flag, unsigned long long target, unsigned long long limit_ns,
                                 KernelStatus* st)
{
    wait_flag_ge(flag, target, st, 100, 0, limit_ns ? limit_ns : kDefaultWaitNs);
}

__global__ void wait_mask_kernel(const unsigned long long* word, unsigned long long mask, unsigned long long limit_ns,
                                 unsigned long long* timed_out)
{
    const unsigned long long lim = limit_ns ? limit_ns : kDefaultWaitNs;
    const unsigned long long t0  = globaltimer_ns();
    while ((ld_acquire_sys(word) & mask) != mask) {
        if (globaltimer_ns() - t0 > lim) {
            // bounded: the stream goes on, and the word tells the host that it did so without the data
            if (timed_out != nullptr) st_release_sys(timed_out, 1ull);
            return;
        }
        __nanosleep(100);
    }
}

__global__ void signal_flag_kernel(unsigned long long* flag, unsigned long long value, int add)
{
    if (add)
        red_add_release_sys(flag, value);
    else
        st_release_sys(flag, value);
}

}  // namespace

extern "C" {

const char* slime_last_error(void)
{
    return last_error_buf();
}

int slime_cuda_version(void)
{
    int v = 0;
    cudaRuntimeGetVersion(&v);
    return v;
}

int slime_status_alloc(void** host_ptr, void** dev_ptr)
{
    void* h = nullptr;
    SLIME_CUDA_OK(cudaHostAlloc(&h, sizeof(KernelStatus), cudaHostAllocMapped | cudaHostAllocPortable));
    memset(h, 0, sizeof(KernelStatus));
    void* d = nullptr;
    SLIME_CUDA_OK(cudaHostGetDevicePointer(&d, h, 0));
    *host_ptr = h;
    *dev_ptr  = d;
    return 0;
}

int slime_status_free(void* host_ptr)
{
    SLIME_CUDA_OK(cudaFreeHost(host_ptr));
    return 0;
}

int slime_host_flags_alloc(unsigned long long n_words, void** host_ptr, void** dev_ptr)
{
    void* h = nullptr;
    SLIME_CUDA_OK(cudaHostAlloc(&h, n_words * 8, cudaHostAllocMapped | cudaHostAllocPortable));
    memset(h, 0, n_words * 8);
    void* d = nullptr;
    SLIME_CUDA_OK(cudaHostGetDevicePointer(&d, h, 0));
    *host_ptr = h;
    *dev_ptr  = d;
    return 0;
}

int slime_host_flags_free(void* host_ptr)
{
    SLIME_CUDA_OK(cudaFreeHost(host_ptr));
    return 0;
}

int slime_wait_flag_kernel(const void* flag, unsigned long long target, unsigned long long limit_ns, void* status,
                           void* stream)
{
    wait_flag_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const unsigned long long*>(flag), target,
                                                                    limit_ns, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_signal_flag_kernel(void* flag, unsigned long long value, int add, void* stream)
{
    signal_flag_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned long long*>(flag), value, add);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

// Stream hooks of the host runtime's stream-ordered signals (see csrc/host/engine/signal.h): word allocation is
// slime_host_flags_alloc / slime_host_flags_free above.
int slime_hook_record_value(void* stream, void* dev_word, unsigned long long value)
{
    signal_flag_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned long long*>(dev_word), value, 0);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_hook_wait_mask(void* stream, void* dev_word, unsigned long long mask, unsigned long long limit_ns,
                         void* dev_timeout_word)
{
    wait_mask_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const unsigned long long*>(dev_word), mask, limit_ns,
                                                                    static_cast<unsigned long long*>(dev_timeout_word));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_symm_alloc(unsigned long long bytes, void** ptr, unsigned char* ipc_handle_out64)
{
    void* p = nullptr;
    SLIME_CUDA_OK(cudaMalloc(&p, bytes));
    SLIME_CUDA_OK(cudaMemset(p, 0, bytes));
    if (ipc_handle_out64) {
        cudaIpcMemHandle_t h;
        cudaError_t        e = cudaIpcGetMemHandle(&h, p);
        if (e != cudaSuccess) {
            cudaFree(p);
            return fail("cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
        }
        static_assert(sizeof(h) == 64, "CUDA IPC handle is 64 bytes");
        memcpy(ipc_handle_out64, &h, 64);
    }
    *ptr = p;
    return 0;
}

int slime_symm_free(void* ptr)
{
    SLIME_CUDA_OK(cudaFree(ptr));
    return 0;
}

int slime_ipc_get_handle(const void* ptr, unsigned char* ipc_handle_out64, unsigned long long* offset_out,
                         unsigned long long* alloc_size_out)
{
    typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
    static RangeFn range_fn = nullptr;
    if (!range_fn) {
        void*                           p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) == cudaSuccess
            && q == cudaDriverEntryPointSuccess)
            range_fn = reinterpret_cast<RangeFn>(p);
    }
    if (!range_fn) return fail("cuMemGetAddressRange entry point not available");
    // The export must run with the device that owns the memory current; callers (agent threads, for one) may have
    // another device current, so the owner is looked up and made current for the two calls.
    int                   cur = 0, owner = -1;
    cudaPointerAttributes attr{};
    SLIME_CUDA_OK(cudaGetDevice(&cur));
    if (cudaPointerGetAttributes(&attr, ptr) == cudaSuccess && attr.type == cudaMemoryTypeDevice) owner = attr.device;
    cudaGetLastError();
    struct Restore {
        int dev;
        bool on;
        ~Restore() { if (on) cudaSetDevice(dev); }
    } restore{cur, false};
    if (owner >= 0 && owner != cur) {
        SLIME_CUDA_OK(cudaSetDevice(owner));
        restore.on = true;
    }
    CUdeviceptr base = 0;
    size_t      size = 0;
    CUresult    r    = range_fn(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
    if (r != CUDA_SUCCESS) return fail("cuMemGetAddressRange failed with CUresult %d", static_cast<int>(r));
    cudaIpcMemHandle_t h;
    SLIME_CUDA_OK(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
    memcpy(ipc_handle_out64, &h, 64);
    if (offset_out) *offset_out = reinterpret_cast<unsigned long long>(ptr) - static_cast<unsigned long long>(base);
    if (alloc_size_out) *alloc_size_out = size;
    return 0;
}

int slime_ipc_open(const unsigned char* ipc_handle64, void** ptr_out)
{
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle64, 64);
    void* p = nullptr;
    SLIME_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr_out = p;
    return 0;
}

int slime_ipc_close(void* ptr)
{
    SLIME_CUDA_OK(cudaIpcCloseMemHandle(ptr));
    return 0;
}

int slime_enable_peer_access(int peer_device)
{
    cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        return 0;
    }
    SLIME_CUDA_OK(e);
    return 0;
}

// Plain cudaMemcpyAsync between two device addresses (local or peer-mapped): the per-segment copy that
// benchmarks use as the baseline for the batched kernels.
int slime_memcpy_async(void* dst, const void* src, unsigned long long bytes, void* stream)
{
    SLIME_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
    return 0;
}

int slime_memset_async(void* ptr, int value, unsigned long long bytes, void* stream)
{
    SLIME_CUDA_OK(cudaMemsetAsync(ptr, value, bytes, static_cast<cudaStream_t>(stream)));
    return 0;
}

}  // extern "C"
