// bf16 GEMM entry points built on the tcgen05 main loop: a plain GEMM (the
// synthetic prefill stand-in), a grouped GEMM over device-side row groups (the
// expert FFN), its SwiGLU-fused variant, and a variant whose epilogue scatters
// weighted rows to arbitrary (possibly peer) addresses.
#include "common/gemm_tc.cuh"
#include "common/host_utils.h"
#include "slime_cuda.h"

using namespace slime;
using namespace slime::gemm;

namespace {

constexpr int kBN     = 256;
constexpr int kStages = 4;

template<int EPI>
int launch(const void* A, const void* B, const Args& args, long long lda, long long ldb, int grid_cap,
           cudaStream_t stream)
{
    using S = Smem<kBN, kStages>;
    CUtensorMap tmA, tmB;
    const unsigned long long rowsB_total = static_cast<unsigned long long>(args.rowsB) * args.num_groups;
    if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.M_total, args.K, lda, kBM, kBK)) return -1;
    if (make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rowsB_total, args.K, ldb, kBN / 2, kBK)) return -1;
    auto kern = gemm_bf16_tc_kernel<kBN, kStages, EPI>;
    static bool configured = false;
    if (!configured) {
        SLIME_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured = true;
    }
    int grid = sm_count();
    if (grid_cap > 0 && grid_cap < grid) grid = grid_cap;
    kern<<<grid, kThreads, S::kTotal, stream>>>(tmA, tmB, args);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

template<bool FUSED>
int launch_ag(const void* A, const void* B, const Args& args, long long lda, long long ldb, int grid_cap, cudaStream_t stream)
{
    using S = Smem<kBN, kStages>;
    CUtensorMap tmA, tmB;
    if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.M_total, args.K, lda, kBM, kBK)) return -1;
    if (make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.rowsB, args.K, ldb, kBN / 2, kBK)) return -1;
    auto kern = gemm_bf16_tc_kernel<kBN, kStages, kEpiStore, FUSED>;
    static bool configured = false;
    if (!configured) {
        SLIME_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured = true;
    }
    int grid = sm_count();
    if (grid_cap > 0 && grid_cap < grid) grid = grid_cap;
    kern<<<grid, kThreads + (FUSED ? kAgThreads : 0), S::kTotal, stream>>>(tmA, tmB, args);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int check_common(int M, int N, int K, long long lda, long long ldb)
{
    if (M <= 0 || N <= 0 || K <= 0) return fail("gemm: M, N, K must be positive (got %d, %d, %d)", M, N, K);
    if (K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0) return fail("gemm: K, lda, ldb must be multiples of 8 elements");
    if (N % 32 != 0) return fail("gemm: N must be a multiple of 32");
    return 0;
}

}  // namespace

extern "C" {

int slime_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                    long long ldc, void* status, void* stream)
{
    if (check_common(M, N, K, lda, ldb)) return -1;
    if (ldc % 8 != 0) return fail("gemm: ldc must be a multiple of 8 elements");
    Args a{};
    a.M_total    = M;
    a.N          = N;
    a.K          = K;
    a.rowsB      = N;
    a.num_groups = 1;
    a.C          = static_cast<__nv_bfloat16*>(C);
    a.ldc        = ldc;
    a.status     = static_cast<KernelStatus*>(status);
    const int tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
    return launch<kEpiStore>(A, B, a, lda, ldb, tiles, static_cast<cudaStream_t>(stream));
}

int slime_gemm_bf16_gated(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, const void* a_ready, int a_ready_rows, unsigned long long a_ready_target,
                          int m_tile_rotate, void* status, void* stream)
{
    if (check_common(M, N, K, lda, ldb)) return -1;
    if (a_ready && (a_ready_rows <= 0)) return fail("gemm: a_ready_rows must be positive");
    Args a{};
    a.M_total        = M;
    a.N              = N;
    a.K              = K;
    a.rowsB          = N;
    a.num_groups     = 1;
    a.C              = static_cast<__nv_bfloat16*>(C);
    a.ldc            = ldc;
    a.a_ready        = static_cast<const unsigned long long*>(a_ready);
    a.a_ready_rows   = a_ready_rows;
    a.a_ready_target = a_ready_target;
    a.m_tile_rotate  = m_tile_rotate;
    a.status         = static_cast<KernelStatus*>(status);
    const int tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
    return launch<kEpiStore>(A, B, a, lda, ldb, tiles, static_cast<cudaStream_t>(stream));
}

// All-gather -> GEMM. a_full is this rank's gathered matrix [world * rows_local, K] inside its symmetric
// region; dst8 / flags8 give the address of that matrix and of its arrival counters on every rank.
// mode 0: push only (separate kernel); 1: GEMM only, gated on the counters; 2: one fused kernel in
// which extra warps push this rank's shard while the tensor-core warps work through the tiles.
int slime_ag_gemm(int mode, const void* x_local, const void* a_full, const void* B, void* C, int rows_local, int N,
                  int K, long long ldb, long long ldc, int rank, int world, const unsigned long long* dst8,
                  const unsigned long long* flags8, unsigned long long step, int push_blocks, void* status,
                  void* stream)
{
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail("ag_gemm: bad rank/world");
    if (rows_local <= 0 || rows_local % kBM != 0) return fail("ag_gemm: rows per rank (%d) must be a multiple of %d", rows_local, kBM);
    if (K % 8 != 0) return fail("ag_gemm: K must be a multiple of 8");
    Args a{};
    a.M_total    = rows_local * world;
    a.N          = N;
    a.K          = K;
    a.rowsB      = N;
    a.num_groups = 1;
    a.C          = static_cast<__nv_bfloat16*>(C);
    a.ldc        = ldc;
    a.status     = static_cast<KernelStatus*>(status);
    a.ag_rows    = rows_local;
    a.ag_rank    = rank;
    a.ag_world   = world;
    for (int i = 0; i < 8; ++i) {
        a.ag_dst[i]   = i < world ? dst8[i] : 0;
        a.ag_flags[i] = i < world ? flags8[i] : 0;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (mode == 0 || mode == 2) {
        if ((reinterpret_cast<unsigned long long>(x_local) & 15) != 0) return fail("ag_gemm: local shard must be 16-byte aligned");
        a.ag_src = static_cast<const uint4*>(x_local);
    }
    if (mode == 0) {
        int grid = push_blocks > 0 ? push_blocks : 32;
        ag_push_only_kernel<<<grid, 256, 0, s>>>(a);
        SLIME_CUDA_OK(cudaGetLastError());
        return 0;
    }
    if (check_common(a.M_total, N, K, K, ldb)) return -1;
    a.a_ready        = reinterpret_cast<const unsigned long long*>(flags8[rank]);
    a.a_ready_rows   = kBM;
    a.a_ready_target = step * (kBM / kAgSliceRows);
    a.ag_shard_order = 1;
    const int tiles = ((a.M_total + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
    if (mode == 1) return launch_ag<false>(a_full, B, a, K, ldb, tiles, s);
    if (mode == 2) return launch_ag<true>(a_full, B, a, K, ldb, 0, s);
    return fail("ag_gemm: unknown mode %d", mode);
}

int slime_grouped_gemm_bf16(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                            int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                            const void* row_info, const unsigned long long* scatter_bases8,
                            unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                            const float* row_scale, void* status, void* stream)
{
    if (check_common(M_cap, N, K, lda, ldb)) return -1;
    if (num_groups <= 0 || group_offsets == nullptr) return fail("grouped gemm: need group offsets");
    Args a{};
    a.M_total       = M_cap;
    a.N             = N;
    a.K             = K;
    a.num_groups    = num_groups;
    a.group_offsets = group_offsets;
    a.C             = static_cast<__nv_bfloat16*>(C);
    a.ldc           = ldc;
    a.status        = static_cast<KernelStatus*>(status);
    cudaStream_t s  = static_cast<cudaStream_t>(stream);
    switch (epilogue) {
        case kEpiStore:
            a.rowsB = N;
            return launch<kEpiStore>(A, B, a, lda, ldb, 0, s);
        case kEpiSwiGLU:
            if (N % (kBN / 2) != 0) return fail("grouped gemm: SwiGLU needs N to be a multiple of %d", kBN / 2);
            a.rowsB = 2 * N;
            return launch<kEpiSwiGLU>(A, B, a, lda, ldb, 0, s);
        case kEpiScatterRows:
            if (row_info == nullptr || scatter_bases8 == nullptr) return fail("grouped gemm: scatter epilogue needs row_info and bases");
            if (scatter_row_bytes % 16 != 0) return fail("grouped gemm: scatter rows must be 16-byte aligned");
            a.rowsB     = N;
            a.row_info  = static_cast<const unsigned long long*>(row_info);
            a.row_scale = row_scale;
            for (int i = 0; i < 8; ++i) a.scatter_base[i] = scatter_bases8[i];
            a.scatter_row_bytes = scatter_row_bytes;
            a.scatter_slots     = scatter_slots;
            return launch<kEpiScatterRows>(A, B, a, lda, ldb, 0, s);
        default:
            return fail("grouped gemm: unknown epilogue %d", epilogue);
    }
}

}  // extern "C"
