// Host-side helpers shared by the kernel launchers: error reporting through a
// thread-local message (the C API returns 0 on success, a negative number on
// error), and TMA tensor-map encoding through the driver entry point so that the
// library needs no link-time dependency on libcuda.
#pragma once

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cuda.h>
#include <cuda_runtime.h>

namespace slime {

inline char* last_error_buf()
{
    static thread_local char buf[512] = {0};
    return buf;
}

inline int fail(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buf(), 512, fmt, ap);
    va_end(ap);
    return -1;
}

#define SLIME_CUDA_OK(expr)                                                                                            \
    do {                                                                                                               \
        cudaError_t _e = (expr);                                                                                       \
        if (_e != cudaSuccess) return ::slime::fail("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void*                            p = nullptr;
        cudaDriverEntryPointQueryResult  q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess
            && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2D row-major matrix [rows, cols] of `elem_bytes`-wide elements with leading
// dimension ld (elements); box = [box_rows, box_cols]; 128-byte swizzle when the
// box row is 128 bytes wide, none otherwise.
inline int make_tmap_2d(CUtensorMap* tm, const void* base, CUtensorMapDataType dt, int elem_bytes,
                        unsigned long long rows, unsigned long long cols, unsigned long long ld,
                        unsigned box_rows, unsigned box_cols)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail("cuTensorMapEncodeTiled entry point not available");
    if ((reinterpret_cast<unsigned long long>(base) & 15) != 0) return fail("TMA base address must be 16-byte aligned");
    if ((ld * elem_bytes) % 16 != 0) return fail("TMA row pitch must be a multiple of 16 bytes");
    cuuint64_t dims[2]    = {cols, rows};
    cuuint64_t strides[1] = {ld * elem_bytes};
    cuuint32_t box[2]     = {box_cols, box_rows};
    cuuint32_t estr[2]    = {1, 1};
    const bool sw128      = box_cols * elem_bytes == 128;
    CUresult   r          = fn(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    sw128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    return 0;
}

// For copy kernels that are meant to run beside the tensor-core GEMMs. A GEMM CTA needs almost all of an SM's shared
// memory, and an SM can only change its split between L1 and shared memory while it is empty: a small kernel that
// leaves the split at "mostly L1" keeps the GEMM's CTA off its SM until its last block there has left (seen as GEMM
// CTAs starting hundreds of microseconds late). Asking for the largest shared-memory split costs a streaming copy
// kernel nothing. Once per device and kernel.
template<typename K>
inline cudaError_t prefer_max_shared_carveout(K kernel, bool (&done)[64])
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess) done[dev] = true;
    return e;
}

// Launches `kernel` so that it may start before the kernel in front of it in `stream` has finished (programmatic
// dependent launch; see griddep_launch_dependents in ptx.cuh).
template<typename... KArgs, typename... Args>
inline cudaError_t launch_programmatic(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                       Args&&... args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = grid;
    cfg.blockDim         = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs                                          = attr;
    cfg.numAttrs                                       = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Multiprocessor count of the current device (cached per device ordinal: a process may drive several GPUs).
inline int sm_count()
{
    constexpr int kMaxDev = 64;
    static int    cached[kMaxDev] = {0};
    int           dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDev) dev = 0;
    int n = cached[dev];
    if (n == 0) {
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
        cached[dev] = n;
    }
    return n;
}

}  // namespace slime
