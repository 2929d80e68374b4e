// Entry points of the block-scaled fp8 GEMM (common/gemm_fp8.cuh): the plain product and the
// all-gather -> GEMM built on it (fp8 payload and scales cross NVLink, half the bytes of the bf16 form).
#include "common/gemm_fp8.cuh"
#include "common/host_utils.h"
#include "slime_cuda.h"

using namespace slime;
using namespace slime::gemm;

namespace {

// Push-only kernel of the all-gather form (single-GPU replay of multi-rank runs, and the unfused baseline).
__global__ void __launch_bounds__(32) ag_push_only_f8_kernel(const F8Args f)
{
    __shared__ __align__(128) uint8_t bufs[4 * kAgChunkBytes];
    __shared__ uint64_t               bars[4];
    if (threadIdx.x == 0) {
        for (int s = 0; s < 4; ++s) mbar_init(&bars[s], 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0)
        ag_push_bulk_f8(f, bufs, bars, 4, blockIdx.x, gridDim.x, f.ag.status, f.ag.wait_ns ? f.ag.wait_ns : kDefaultWaitNs);
}

template<bool AG>
int launch_f8(const void* Aq, const void* Bq, const void* A_local, const F8Args& f, long long lda, long long ldb, cudaStream_t stream)
{
    using S = SmemF8<AG>;
    CUtensorMap tmA, tmB, tmAL;
    if (make_tmap_2d(&tmA, Aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, f.M, f.K, lda, kBM, kF8BK)) return -1;
    if (make_tmap_2d(&tmB, Bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, f.N, f.K, ldb, kF8BN / 2, kF8BK)) return -1;
    if (A_local) {
        if (make_tmap_2d(&tmAL, A_local, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, f.ag.ag_rows, f.K, f.K, kBM, kF8BK)) return -1;
    }
    else {
        tmAL = tmA;
    }
    auto kern = gemm_fp8_blockscaled_kernel<AG>;
    static bool configured = false;
    if (!configured) {
        SLIME_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured = true;
    }
    const long tiles = static_cast<long>((f.M + kBM - 1) / kBM) * ((f.N + kF8BN - 1) / kF8BN);
    int        grid  = sm_count();
    if (!AG && tiles < grid) grid = static_cast<int>(tiles);
    kern<<<grid, kF8Threads + (AG ? kAgThreads : 0), S::kTotal, stream>>>(tmA, tmB, tmAL, f);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int check_f8(int M, int N, int K, long long lda, long long ldb, long long ldc)
{
    if (M <= 0 || N <= 0 || K <= 0) return fail("fp8 gemm: M, N, K must be positive (got %d, %d, %d)", M, N, K);
    if (K % kF8BK != 0) return fail("fp8 gemm: K (%d) must be a multiple of %d (one scale block)", K, kF8BK);
    if (lda % 16 != 0 || ldb % 16 != 0) return fail("fp8 gemm: lda and ldb must be multiples of 16 bytes");
    if (N % 32 != 0 || ldc % 8 != 0) return fail("fp8 gemm: N must be a multiple of 32 and ldc of 8");
    return 0;
}

}  // namespace

extern "C" {

// C[M, N] (bf16) = dequant(Aq, sa) * dequant(Bq, sb)^T with 1x128 scales for A and 128x128 scales for B.
int slime_gemm_fp8_blockscaled(const void* Aq, const float* sa, const void* Bq, const float* sb, void* C, int M, int N, int K,
                               long long lda, long long ldb, long long ldc, void* status, void* stream)
{
    if (check_f8(M, N, K, lda, ldb, ldc)) return -1;
    F8Args f{};
    f.M = M;
    f.N = N;
    f.K = K;
    f.C = static_cast<__nv_bfloat16*>(C);
    f.ldc = ldc;
    f.sa = sa;
    f.sb = sb;
    f.ag.status = static_cast<KernelStatus*>(status);
    return launch_f8<false>(Aq, Bq, nullptr, f, lda, ldb, static_cast<cudaStream_t>(stream));
}

// All-gather -> GEMM in fp8. xq_local / sx_local: this rank's quantised shard [rows_local, K] and its scales
// [rows_local, K/128]; aq_full / sa_full: this rank's gathered matrices inside its symmetric region; dst8 / sdst8 /
// flags8: the addresses of those two matrices and of the arrival counters on every rank.
// mode 0: push only; 1: GEMM only, gated on the counters; 2: one fused kernel.
int slime_ag_gemm_fp8(int mode, const void* xq_local, const float* sx_local, const void* aq_full, const float* sa_full,
                      const void* Bq, const float* sb, void* C, int rows_local, int N, int K, long long ldb, long long ldc, int rank,
                      int world, const unsigned long long* dst8, const unsigned long long* sdst8, const unsigned long long* flags8,
                      unsigned long long step, int push_blocks, void* status, void* stream)
{
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail("ag_gemm_fp8: bad rank/world");
    if (rows_local <= 0 || rows_local % kBM != 0) return fail("ag_gemm_fp8: rows per rank (%d) must be a multiple of %d", rows_local, kBM);
    if (K % kF8BK != 0) return fail("ag_gemm_fp8: K must be a multiple of %d", kF8BK);
    F8Args f{};
    f.M = rows_local * world;
    f.N = N;
    f.K = K;
    f.C = static_cast<__nv_bfloat16*>(C);
    f.ldc = ldc;
    f.sa = sa_full;
    f.sa_local = sx_local;
    f.sb = sb;
    f.ag.status   = static_cast<KernelStatus*>(status);
    f.ag.ag_rows  = rows_local;
    f.ag.ag_rank  = rank;
    f.ag.ag_world = world;
    for (int i = 0; i < 8; ++i) {
        f.ag.ag_dst[i]     = i < world ? dst8[i] : 0;
        f.ag.ag_flags[i]   = i < world ? flags8[i] : 0;
        f.ag_dst_scales[i] = i < world ? sdst8[i] : 0;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (mode == 0 || mode == 2) {
        if ((reinterpret_cast<unsigned long long>(xq_local) & 15) != 0 || (reinterpret_cast<unsigned long long>(sx_local) & 15) != 0)
            return fail("ag_gemm_fp8: local shard and scales must be 16-byte aligned");
        f.ag.ag_src      = static_cast<const uint4*>(xq_local);
        f.ag_src_scales  = reinterpret_cast<const uint8_t*>(sx_local);
    }
    if (mode == 0) {
        ag_push_only_f8_kernel<<<push_blocks > 0 ? push_blocks : 64, 32, 0, s>>>(f);
        SLIME_CUDA_OK(cudaGetLastError());
        return 0;
    }
    if (check_f8(f.M, N, K, K, ldb, ldc)) return -1;
    f.ag.a_ready        = reinterpret_cast<const unsigned long long*>(flags8[rank]);
    f.ag.a_ready_rows   = kBM;
    f.ag.a_ready_target = step * (kBM / kAgSliceRows);
    f.ag.ag_shard_order = 1;
    if (mode == 1) return launch_f8<false>(aq_full, Bq, nullptr, f, K, ldb, s);
    if (mode == 2) {
        f.ag.ag_local_direct = 1;
        return launch_f8<true>(aq_full, Bq, xq_local, f, K, ldb, s);
    }
    return fail("ag_gemm_fp8: unknown mode %d", mode);
}

}  // extern "C"
