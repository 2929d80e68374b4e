// Block-scaled fp8 e4m3 quantisation and dequantisation.
//   1x128   : one fp32 scale per 128 consecutive elements of a row (activations)
//   128x128 : one fp32 scale per 128x128 tile (weights)
// With c = max(amax, 1e-4): scale = c / 448, q = rne_sat(x * (448 / c)). Vector kernels, bound by
// HBM bandwidth: 16-byte loads, 8-byte fp8 stores, amax by shuffles, one multiply per element.
#include "common/fp8.cuh"
#include "common/host_utils.h"
#include "slime_cuda.h"

using namespace slime;

namespace {

// Dequantisation: 16 lanes cover one 128-element group (8 values each); a warp covers 2 * kGroupsPerLane consecutive
// groups and issues all of its loads before it uses any of them. kContig: both matrices are dense (pitch == cols), so a
// group's offset is its index times 128 and no row / column split (a 64-bit division) is needed.
constexpr int kGroupsPerLane = 2;

template<bool kContig>
__device__ __forceinline__ void group_offsets(long long gid, int groups_per_row, long long ld_a, long long ld_b,
                                              long long& off_a, long long& off_b)
{
    if (kContig) {
        off_a = off_b = gid * 128;
    }
    else {
        const long long row = gid / groups_per_row;
        const long long col = (gid - row * groups_per_row) * 128;
        off_a               = row * ld_a + col;
        off_b               = row * ld_b + col;
    }
}

// Quantisation: 8 lanes per group, each with elements [8 s, 8 s + 8) and [64 + 8 s, 64 + 8 s + 8) of it, so every load
// and store instruction of a warp touches whole 128-byte (64-byte for fp8) runs, and the per-group work (three
// shuffle steps, two divisions) is shared by 16 elements per lane instead of 8. A warp covers 4 * kQuantPasses groups.
constexpr int kQuantPasses = 2;

template<bool kContig>
__global__ void __launch_bounds__(256) quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                         float* __restrict__ scales, long long n_groups,
                                                         int groups_per_row, long long ldx, long long ldq)
{
    const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int       quad = (threadIdx.x >> 3) & 3, sub = threadIdx.x & 7;
    long long       gid[kQuantPasses], ox[kQuantPasses], oq[kQuantPasses];
    uint4           lo[kQuantPasses], hi[kQuantPasses];
#pragma unroll
    for (int j = 0; j < kQuantPasses; ++j) {
        gid[j] = warp * (4 * kQuantPasses) + 4 * j + quad;
        lo[j] = hi[j] = make_uint4(0u, 0u, 0u, 0u);
        if (gid[j] < n_groups) {
            group_offsets<kContig>(gid[j], groups_per_row, ldx, ldq, ox[j], oq[j]);
            lo[j] = *reinterpret_cast<const uint4*>(x + ox[j] + sub * 8);
            hi[j] = *reinterpret_cast<const uint4*>(x + ox[j] + 64 + sub * 8);
        }
    }
#pragma unroll
    for (int j = 0; j < kQuantPasses; ++j) {
        float v[16];
        unpack_bf16x8(lo[j], v);
        unpack_bf16x8(hi[j], v + 8);
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int o = 4; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o, 8));  // all 32 lanes take part
        if (gid[j] < n_groups) {
            const Fp8Scale fs = fp8_scale_from_amax(amax);
            *reinterpret_cast<uint2*>(q + oq[j] + sub * 8)      = quant_fp8x8(v, fs.inv);
            *reinterpret_cast<uint2*>(q + oq[j] + 64 + sub * 8) = quant_fp8x8(v + 8, fs.inv);
            if (sub == 0) scales[gid[j]] = fs.scale;
        }
    }
}

template<bool kContig>
__global__ void __launch_bounds__(256) dequant_1x128_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scales,
                                                           __nv_bfloat16* __restrict__ y, long long n_groups,
                                                           int groups_per_row, long long ldq, long long ldy)
{
    const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int       half = (threadIdx.x >> 4) & 1, sub = threadIdx.x & 15;
    long long       gid[kGroupsPerLane], oq[kGroupsPerLane], oy[kGroupsPerLane];
    uint2           raw[kGroupsPerLane];
    float           scale[kGroupsPerLane];
#pragma unroll
    for (int j = 0; j < kGroupsPerLane; ++j) {
        gid[j] = warp * (2 * kGroupsPerLane) + 2 * j + half;
        if (gid[j] < n_groups) {
            group_offsets<kContig>(gid[j], groups_per_row, ldq, ldy, oq[j], oy[j]);
            raw[j]   = *reinterpret_cast<const uint2*>(q + oq[j] + sub * 8);
            scale[j] = scales[gid[j]];
        }
    }
#pragma unroll
    for (int j = 0; j < kGroupsPerLane; ++j) {
        if (gid[j] < n_groups) {
            float v[8];
            dequant_fp8x8(raw[j], scale[j], v);
            *reinterpret_cast<uint4*>(y + oy[j] + sub * 8) = pack_bf16x8(v);
        }
    }
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
    const Fp8Scale fs = fp8_scale_from_amax(amax);
    if (threadIdx.x == 0) scales[static_cast<long long>(tile_r) * gridDim.x + tile_c] = fs.scale;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = c0 + i * 8;
        if (in && c < cols)
            *reinterpret_cast<uint2*>(q + static_cast<long long>(r) * ldq + c) = quant_fp8x8(v + i * 8, fs.inv);
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
    const long long per_block = 256 / 8 * kQuantPasses;
    const long long blocks    = (n_groups + per_block - 1) / per_block;
    if (blocks > 0x7fffffffLL) return fail("fp8 quant: %lld groups exceed one launch", n_groups);
    auto kernel = (ldx == cols && ldq == cols) ? quant_1x128_kernel<true> : quant_1x128_kernel<false>;
    kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
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
    const long long per_block = 256 / 16 * kGroupsPerLane;
    const long long blocks    = (n_groups + per_block - 1) / per_block;
    if (blocks > 0x7fffffffLL) return fail("fp8 dequant: %lld groups exceed one launch", n_groups);
    auto kernel = (ldq == cols && ldy == cols) ? dequant_1x128_kernel<true> : dequant_1x128_kernel<false>;
    kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
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
