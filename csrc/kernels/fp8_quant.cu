// Block-scaled fp8 e4m3 quantisation and dequantisation.
//   1x128   : one fp32 scale per 128 consecutive elements of a row (activations)
//   128x128 : one fp32 scale per 128x128 tile (weights)
// scale = max(amax, 1e-4) / 448, q = rne_sat(x / scale). Vector kernels, bound by
// HBM bandwidth: 16-byte loads, 8-byte fp8 stores, amax by shuffles.
#include "common/fp8.cuh"
#include "common/host_utils.h"
#include "slime_cuda.h"

using namespace slime;

namespace {

// 16 threads cover one 128-element group (8 bf16 each).
__global__ void __launch_bounds__(256) quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                         float* __restrict__ scales, long long n_groups,
                                                         int groups_per_row, long long ldx, long long ldq)
{
    const long long gid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
    const int       sub = threadIdx.x & 15;
    if (gid >= n_groups) return;  // whole 16-lane segments leave together
    const long long row = gid / groups_per_row;
    const int       grp = static_cast<int>(gid - row * groups_per_row);
    const uint4     raw = *reinterpret_cast<const uint4*>(x + row * ldx + grp * 128 + sub * 8);
    float           v[8];
    unpack_bf16x8(raw, v);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o, 16));
    const float scale = fp8_scale_from_amax(amax);
    *reinterpret_cast<uint2*>(q + row * ldq + grp * 128 + sub * 8) = quant_fp8x8(v, scale);
    if (sub == 0) scales[gid] = scale;
}

__global__ void __launch_bounds__(256) dequant_1x128_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scales,
                                                           __nv_bfloat16* __restrict__ y, long long n_groups,
                                                           int groups_per_row, long long ldq, long long ldy)
{
    const long long gid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
    const int       sub = threadIdx.x & 15;
    if (gid >= n_groups) return;
    const long long row   = gid / groups_per_row;
    const int       grp   = static_cast<int>(gid - row * groups_per_row);
    const uint2     raw   = *reinterpret_cast<const uint2*>(q + row * ldq + grp * 128 + sub * 8);
    const float     scale = scales[gid];
    float           v[8];
    dequant_fp8x8(raw, scale, v);
    *reinterpret_cast<uint4*>(y + row * ldy + grp * 128 + sub * 8) = pack_bf16x8(v);
}

// One CTA (256 threads) per 128x128 tile: thread t handles row t/2, 64 columns.
__global__ void __launch_bounds__(256) quant_128x128_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                                                           float* __restrict__ scales, int rows, int cols,
                                                           long long ldw, long long ldq)
{
    __shared__ float warp_max[8];
    const int tile_c = blockIdx.x, tile_r = blockIdx.y;
    const int r      = tile_r * 128 + (threadIdx.x >> 1);
    const int c0     = tile_c * 128 + (threadIdx.x & 1) * 64;
    float     v[64];
    float     amax = 0.f;
    const bool in  = r < rows;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = c0 + i * 8;
        if (in && c < cols) {
            const uint4 raw = *reinterpret_cast<const uint4*>(w + static_cast<long long>(r) * ldw + c);
            unpack_bf16x8(raw, v + i * 8);
        }
        else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i * 8 + j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[i * 8 + j]));
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = warp_max[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, warp_max[i]);
    const float scale = fp8_scale_from_amax(amax);
    if (threadIdx.x == 0) scales[static_cast<long long>(tile_r) * gridDim.x + tile_c] = scale;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = c0 + i * 8;
        if (in && c < cols)
            *reinterpret_cast<uint2*>(q + static_cast<long long>(r) * ldq + c) = quant_fp8x8(v + i * 8, scale);
    }
}

}  // namespace

extern "C" {

int slime_fp8_quant_1x128(const void* x, void* q, float* scales, long long rows, int cols, long long ldx,
                          long long ldq, void* stream)
{
    if (cols <= 0 || cols % 128 != 0) return fail("fp8 quant: cols (%d) must be a positive multiple of 128", cols);
    if (ldx % 8 != 0 || ldq % 8 != 0) return fail("fp8 quant: row pitches must be multiples of 8 elements");
    if (rows <= 0) return 0;
    const long long n_groups = rows * (cols / 128);
    const long long blocks   = (n_groups * 16 + 255) / 256;
    quant_1x128_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scales, n_groups, cols / 128, ldx, ldq);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_fp8_dequant_1x128(const void* q, const float* scales, void* y, long long rows, int cols, long long ldq,
                            long long ldy, void* stream)
{
    if (cols <= 0 || cols % 128 != 0) return fail("fp8 dequant: cols (%d) must be a positive multiple of 128", cols);
    if (ldy % 8 != 0 || ldq % 8 != 0) return fail("fp8 dequant: row pitches must be multiples of 8 elements");
    if (rows <= 0) return 0;
    const long long n_groups = rows * (cols / 128);
    const long long blocks   = (n_groups * 16 + 255) / 256;
    dequant_1x128_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(q), scales, static_cast<__nv_bfloat16*>(y), n_groups, cols / 128, ldq, ldy);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_fp8_quant_128x128(const void* w, void* q, float* scales, int rows, int cols, long long ldw, long long ldq,
                            void* stream)
{
    if (rows <= 0 || cols <= 0) return fail("fp8 weight quant: empty matrix");
    if (cols % 8 != 0 || ldw % 8 != 0 || ldq % 8 != 0) return fail("fp8 weight quant: cols and pitches must be multiples of 8");
    dim3 grid((cols + 127) / 128, (rows + 127) / 128);
    quant_128x128_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q), scales, rows, cols, ldw, ldq);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

}  // extern "C"
