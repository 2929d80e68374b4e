// bf16 GEMM entry points built on the tcgen05 main loop: a plain GEMM (the
// synthetic prefill stand-in), a grouped GEMM over device-side row groups (the
// expert FFN), its SwiGLU-fused variant, and a variant whose epilogue scatters
// weighted rows to arbitrary (possibly peer) addresses.
#include "common/gemm_tc2s.cuh"
#include "common/gemm_tc2w.cuh"
#include "common/host_utils.h"
#include "slime_cuda.h"

using namespace slime;
using namespace slime::gemm;

namespace {

constexpr int kBN     = 256;
constexpr int kStages = 4;

// Tile width for one-group GEMMs: the widest tile wins unless a narrower one saves whole waves of the
// persistent grid (cost = waves x (width + a fixed per-tile overhead expressed in columns)).
int pick_bn(int M, int N)
{
    const int  sms    = sm_count();
    const long mtiles = (M + kBM - 1) / kBM;
    int        best = 256;
    long       best_cost = -1;
    for (int bn : {256, 224, 192}) {
        const long tiles = mtiles * ((N + bn - 1) / bn);
        const long cost  = ((tiles + sms - 1) / sms) * (bn + 12);
        if (best_cost < 0 || cost < best_cost) {
            best      = bn;
            best_cost = cost;
        }
    }
    return best;
}

template<int BN, int EPI, bool AG, int AROWS = kBM, int STAGES = kStages>
int launch_bn(const void* A, const void* B, const void* A_local, int rows_local, const Args& args, long long lda, long long ldb,
              int threads, cudaStream_t stream)
{
    using S = Smem<BN, STAGES, AG, false, AROWS>;
    CUtensorMap tmA, tmB, tmAL;
    const unsigned long long rowsB_total = static_cast<unsigned long long>(args.rowsB) * args.num_groups;
    if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.M_total, args.K, lda, AROWS, kBK)) return -1;
    if (make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rowsB_total, args.K, ldb, BN / 2, kBK)) return -1;
    if (A_local) {
        if (make_tmap_2d(&tmAL, A_local, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_local, args.K, args.K, kBM, kBK)) return -1;
    }
    else {
        tmAL = tmA;
    }
    auto kern = gemm_bf16_tc_kernel<BN, STAGES, EPI, AG, false, AROWS>;
    static bool configured = false;
    if (!configured) {
        SLIME_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured = true;
    }
    const long tiles = static_cast<long>((args.M_total + AROWS - 1) / AROWS) * ((args.N + BN - 1) / BN);
    int        grid  = sm_count();
    // a fused all-gather kernel keeps the full grid (its extra warps push whatever the tile count is);
    // grouped launches do not know their tile count on the host
    if (!AG && args.num_groups == 1 && tiles < grid) grid = static_cast<int>(tiles);
    if (args.group_ready != nullptr) {
        // groups that are filled while this kernel runs: start beside the kernel in front of it in the stream
        SLIME_CUDA_OK(launch_programmatic(kern, dim3(grid), dim3(threads), S::kTotal, stream, tmA, tmB, tmAL, args));
        return 0;
    }
    kern<<<grid, threads, S::kTotal, stream>>>(tmA, tmB, tmAL, args);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

thread_local int g_tile_n     = 0;  // set around one grouped launch on single CTAs: tile width 128 / 192 / 224 (0 = 256)
thread_local int g_w_prefetch = 0;  // and the distance of its weight prefetch in K blocks (0 = none)
thread_local int g_tile_m     = 0;  // 64: row tiles of 64 with a five-stage ring (groups of a few dozen rows)

template<int EPI>
int launch(const void* A, const void* B, const Args& args, long long lda, long long ldb, cudaStream_t stream)
{
    // A grouped launch with few tiles (decode-size steps on many ranks: 32 experts x 16 tile columns = 3.46 waves of 148)
    // is quantised by the wave count; the caller, who knows the expected number of row tiles, may ask for a narrower tile.
    if (args.group_ready == nullptr && g_tile_m == 64 && g_tile_n == 0)
        return launch_bn<kBN, EPI, false, 64, 5>(A, B, nullptr, 0, args, lda, ldb, kThreads, stream);
    if (args.group_ready == nullptr) {
        switch (g_tile_n) {
            case 128: return launch_bn<128, EPI, false>(A, B, nullptr, 0, args, lda, ldb, kThreads, stream);
            case 192: return launch_bn<192, EPI, false>(A, B, nullptr, 0, args, lda, ldb, kThreads, stream);
            case 224: return launch_bn<224, EPI, false>(A, B, nullptr, 0, args, lda, ldb, kThreads, stream);
            default: break;
        }
    }
    if (EPI == kEpiStore && args.num_groups == 1) {
        switch (pick_bn(args.M_total, args.N)) {
            case 224: return launch_bn<224, kEpiStore, false>(A, B, nullptr, 0, args, lda, ldb, kThreads, stream);
            case 192: return launch_bn<192, kEpiStore, false>(A, B, nullptr, 0, args, lda, ldb, kThreads, stream);
            default: break;
        }
    }
    return launch_bn<kBN, EPI, false>(A, B, nullptr, 0, args, lda, ldb, kThreads, stream);
}

template<bool FUSED>
int launch_ag(const void* A, const void* B, const void* A_local, const Args& args, long long lda, long long ldb, cudaStream_t stream)
{
    const int threads = kThreads + (FUSED ? kAgThreads : 0);
    switch (pick_bn(args.M_total, args.N)) {
        case 224: return launch_bn<224, kEpiStore, FUSED>(A, B, A_local, args.ag_rows, args, lda, ldb, threads, stream);
        case 192: return launch_bn<192, kEpiStore, FUSED>(A, B, A_local, args.ag_rows, args, lda, ldb, threads, stream);
        default: return launch_bn<kBN, kEpiStore, FUSED>(A, B, A_local, args.ag_rows, args, lda, ldb, threads, stream);
    }
}

// Grouped GEMM whose A operand is e4m3 with 1x128 scales, expanded to bf16 inside the kernel (three stages: the raw
// tile needs room next to the bf16 one).
template<int EPI>
int launch_a8(const void* Aq, const void* B, const Args& args, long long lda_bytes, long long ldb, cudaStream_t stream)
{
    constexpr int kStagesA8 = 3;
    using S = Smem<kBN, kStagesA8, false, true>;
    CUtensorMap tmA, tmB;
    const unsigned long long rowsB_total = static_cast<unsigned long long>(args.rowsB) * args.num_groups;
    if (make_tmap_2d(&tmA, Aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, args.M_total, args.K, lda_bytes, kBM, kBK)) return -1;
    if (make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rowsB_total, args.K, ldb, kBN / 2, kBK)) return -1;
    auto kern = gemm_bf16_tc_kernel<kBN, kStagesA8, EPI, false, true>;
    static bool configured = false;
    if (!configured) {
        SLIME_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured = true;
    }
    kern<<<sm_count(), kThreads + kCvtThreads, S::kTotal, stream>>>(tmA, tmB, tmA, args);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

// CTA-pair kernels: 256-row tiles on clusters of two CTAs (one-group GEMMs only).
int pick_bn_pair(int M, int N)
{
    const int  clusters = sm_count() / 2;
    const long mtiles   = (M + kPairBM - 1) / kPairBM;
    int        best = 256;
    long       best_cost = -1;
    for (int bn : {256, 224, 192}) {
        const long tiles = mtiles * ((N + bn - 1) / bn);
        const long cost  = ((tiles + clusters - 1) / clusters) * (bn + 12);
        if (best_cost < 0 || cost < best_cost) {
            best      = bn;
            best_cost = cost;
        }
    }
    return best;
}

template<int BN, int STAGES, bool AG>
int launch_pair_bn(const void* A, const void* B, const void* A_local, const Args& args, long long lda, long long ldb, cudaStream_t stream)
{
    using S = SmemPair<BN, STAGES, AG>;
    CUtensorMap tmA, tmB, tmAL;
    if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.M_total, args.K, lda, kBM, kBK)) return -1;
    if (make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.rowsB, args.K, ldb, BN / 2, kBK)) return -1;
    if (A_local) {
        if (make_tmap_2d(&tmAL, A_local, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.ag_rows, args.K, args.K, kBM, kBK)) return -1;
    }
    else {
        tmAL = tmA;
    }
    auto kern = gemm_bf16_pair_kernel<BN, STAGES, AG>;
    static bool configured = false;
    if (!configured) {
        SLIME_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured = true;
    }
    const long tiles    = static_cast<long>((args.M_total + kPairBM - 1) / kPairBM) * ((args.N + BN - 1) / BN);
    int        clusters = sm_count() / 2;
    if (!AG && tiles < clusters) clusters = static_cast<int>(tiles);
    kern<<<2 * clusters, kThreads + (AG ? kAgThreads : 0), S::kTotal, stream>>>(tmA, tmB, tmAL, args);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

template<bool AG>
int launch_pair(const void* A, const void* B, const void* A_local, const Args& args, long long lda, long long ldb, cudaStream_t stream)
{
    switch (pick_bn_pair(args.M_total, args.N)) {
        case 224: return launch_pair_bn<224, 6, AG>(A, B, A_local, args, lda, ldb, stream);
        case 192: return launch_pair_bn<192, 7, AG>(A, B, A_local, args, lda, ldb, stream);
        default: return launch_pair_bn<256, 6, AG>(A, B, A_local, args, lda, ldb, stream);
    }
}

// The grouped GEMM on CTA pairs: 256-row tiles per group, every epilogue of the single-CTA kernel.
template<int EPI>
int launch_pair_grouped(const void* A, const void* B, const Args& args, long long lda, long long ldb, cudaStream_t stream)
{
    constexpr int kPairStages = 6;
    using S = SmemPair<kBN, kPairStages, false>;
    CUtensorMap tmA, tmB;
    const unsigned long long rowsB_total = static_cast<unsigned long long>(args.rowsB) * args.num_groups;
    if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.M_total, args.K, lda, kBM, kBK)) return -1;
    if (make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rowsB_total, args.K, ldb, kBN / 2, kBK)) return -1;
    auto kern = gemm_bf16_pair_grouped_kernel<kBN, kPairStages, EPI>;
    static bool configured = false;
    if (!configured) {
        SLIME_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured = true;
    }
    kern<<<2 * (sm_count() / 2), kThreads, S::kTotal, stream>>>(tmA, tmB, args);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

// CTA pairs with swapped operands: weight rows on the M side, a group's tokens (any multiple of 16 up to 256) on the N side.
template<int EPI>
int launch_pair_swapped(const void* A, const void* B, const Args& args, long long lda, long long ldb, cudaStream_t stream)
{
    constexpr int kSwapStages = 6;
    using S = SmemSwap<kSwapStages>;
    CUtensorMap tmW, tmX;
    const unsigned long long rowsB_total = static_cast<unsigned long long>(args.rowsB) * args.num_groups;
    if (make_tmap_2d(&tmX, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.M_total, args.K, lda, kBM, kBK)) return -1;
    if (make_tmap_2d(&tmW, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rowsB_total, args.K, ldb, EPI == kEpiSwiGLU ? kBM / 2 : kBM, kBK)) return -1;
    auto kern = gemm_bf16_pair_swapped_kernel<kSwapStages, EPI>;
    static bool configured = false;
    if (!configured) {
        SLIME_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured = true;
    }
    kern<<<2 * (sm_count() / 2), kThreads, S::kTotal, stream>>>(tmW, tmX, args);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

// CTA pairs with 256 x 512 tiles (two accumulator blocks): plain (num_groups == 1, no offsets) and grouped GEMMs.
template<int EPI>
int launch_pair_wide(const void* A, const void* B, const Args& args, long long lda, long long ldb, cudaStream_t stream)
{
    constexpr int kWideStages = 4;
    using S = SmemWide<kBN, kWideStages>;
    CUtensorMap tmA, tmB;
    const unsigned long long rowsB_total = static_cast<unsigned long long>(args.rowsB) * args.num_groups;
    if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, args.M_total, args.K, lda, kBM, kBK)) return -1;
    if (make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rowsB_total, args.K, ldb, kBN / 2, kBK)) return -1;
    auto kern = gemm_bf16_pair_wide_kernel<kBN, kWideStages, EPI>;
    static bool configured = false;
    if (!configured) {
        SLIME_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured = true;
    }
    int clusters = sm_count() / 2;
    if (args.group_offsets == nullptr) {
        constexpr int kTileOut = EPI == kEpiSwiGLU ? kBN : 2 * kBN;
        const long    tiles    = static_cast<long>((args.M_total + kPairBM - 1) / kPairBM) * ((args.N + kTileOut - 1) / kTileOut);
        if (tiles < clusters) clusters = static_cast<int>(tiles);
    }
    kern<<<2 * clusters, kWideThreads, S::kTotal, stream>>>(tmA, tmB, args);
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
    return launch<kEpiStore>(A, B, a, lda, ldb, static_cast<cudaStream_t>(stream));
}

// The same product on CTA pairs (256-row tiles, tcgen05 cta_group::2).
int slime_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
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
    return launch_pair<false>(A, B, nullptr, a, lda, ldb, static_cast<cudaStream_t>(stream));
}

// The same on CTA pairs with 256 x 512 tiles and a tile order that keeps a band of B rows in L2.
int slime_gemm_bf16_wide(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
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
    return launch_pair_wide<kEpiStore>(A, B, a, lda, ldb, static_cast<cudaStream_t>(stream));
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
    return launch<kEpiStore>(A, B, a, lda, ldb, static_cast<cudaStream_t>(stream));
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
    if (mode == 0 || mode == 2 || mode == 3) {
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
    if (mode == 1) return launch_ag<false>(a_full, B, nullptr, a, K, ldb, s);
    a.ag_local_direct = 1;
    if (mode == 2) return launch_ag<true>(a_full, B, x_local, a, K, ldb, s);
    if (mode == 3) {  // fused, on CTA pairs
        if (rows_local % kPairBM != 0) return fail("ag_gemm: the pair kernel needs rows per rank to be a multiple of %d", kPairBM);
        return launch_pair<true>(a_full, B, x_local, a, K, ldb, s);
    }
    return fail("ag_gemm: unknown mode %d", mode);
}

static int grouped_gemm_impl(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                            int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                            const void* row_info, const unsigned long long* scatter_bases8,
                            unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                            const float* row_scale, const unsigned long long* group_ready,
                            unsigned long long group_ready_target, const unsigned long long* group_ready_epoch,
                            void* status, void* stream);
static thread_local unsigned long long* g_group_trace  = nullptr;  // set around one traced launch
static thread_local unsigned int*       g_tile_counter = nullptr;
static thread_local int                 g_on_pairs     = 0;  // set around one launch on CTA pairs: 1 = 256 x 256 tiles, 2 = 256 x 512
int slime_grouped_gemm_bf16_gated_traced(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                         int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                         const void* group_ready, unsigned long long group_ready_target,
                                         const void* group_ready_epoch, void* group_trace, void* tile_counter, void* status,
                                         void* stream);

int slime_grouped_gemm_bf16(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                            int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                            const void* row_info, const unsigned long long* scatter_bases8,
                            unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                            const float* row_scale, void* status, void* stream)
{
    return grouped_gemm_impl(A, B, C, group_offsets, num_groups, M_cap, N, K, lda, ldb, ldc, epilogue, row_info, scatter_bases8,
                             scatter_row_bytes, scatter_slots, row_scale, nullptr, 0, nullptr, status, stream);
}

// The same on single CTAs with options: a tile width of 128, 192 or 224 columns instead of 256 (SwiGLU: half of it in
// output columns), a weight prefetch into L2 w_prefetch K blocks ahead of the loads (for launches with few rows per
// group, which stream their weights from HBM), and row tiles of 64 (tile_m = 64): the A part of a stage shrinks from 16
// to 8 KB, which makes room for a fifth stage, i.e. 160 instead of 128 KB of weight tiles in flight per SM.
int slime_grouped_gemm_bf16_tile(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                 int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                 const void* row_info, const unsigned long long* scatter_bases8,
                                 unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                                 const float* row_scale, int tile_n, int w_prefetch, int tile_m, void* status, void* stream)
{
    if (tile_m != 0 && tile_m != 64 && tile_m != 128) return fail("grouped gemm: row tiles of %d are not offered", tile_m);
    if (tile_m == 64 && tile_n != 0 && tile_n != 256) return fail("grouped gemm: row tiles of 64 come with 256-wide tiles only");
    g_tile_m = tile_m == 64 ? 64 : 0;
    if (tile_n != 0 && tile_n != 128 && tile_n != 192 && tile_n != 224 && tile_n != 256) return fail("grouped gemm: tile width %d is not offered", tile_n);
    if (w_prefetch < 0 || w_prefetch > 64) return fail("grouped gemm: weight prefetch distance %d not in [0, 64]", w_prefetch);
    g_tile_n     = tile_n == 256 ? 0 : tile_n;
    g_w_prefetch = w_prefetch;
    const int rc = grouped_gemm_impl(A, B, C, group_offsets, num_groups, M_cap, N, K, lda, ldb, ldc, epilogue, row_info, scatter_bases8,
                                     scatter_row_bytes, scatter_slots, row_scale, nullptr, 0, nullptr, status, stream);
    g_tile_n     = 0;
    g_w_prefetch = 0;
    g_tile_m     = 0;
    return rc;
}

// The same on CTA pairs (256-row tiles; pays off for groups of several hundred rows and more).
int slime_grouped_gemm_bf16_pair(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                 int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                 const void* row_info, const unsigned long long* scatter_bases8,
                                 unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                                 const float* row_scale, void* status, void* stream)
{
    g_on_pairs   = 1;
    const int rc = grouped_gemm_impl(A, B, C, group_offsets, num_groups, M_cap, N, K, lda, ldb, ldc, epilogue, row_info, scatter_bases8,
                                     scatter_row_bytes, scatter_slots, row_scale, nullptr, 0, nullptr, status, stream);
    g_on_pairs   = 0;
    return rc;
}

// The same on CTA pairs with the operands swapped (weights on the M side of the MMA, a group's tokens on the N side in
// steps of 16): no rows are computed for nothing and a group of up to 256 rows reads its weights once.
int slime_grouped_gemm_bf16_swapped(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                    int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                    const void* row_info, const unsigned long long* scatter_bases8,
                                    unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                                    const float* row_scale, void* status, void* stream)
{
    if (ldc % 4 != 0 || scatter_row_bytes % 8 != 0) return fail("swapped grouped gemm: rows of the output must be 8-byte aligned");
    g_on_pairs   = 3;
    const int rc = grouped_gemm_impl(A, B, C, group_offsets, num_groups, M_cap, N, K, lda, ldb, ldc, epilogue, row_info, scatter_bases8,
                                     scatter_row_bytes, scatter_slots, row_scale, nullptr, 0, nullptr, status, stream);
    g_on_pairs   = 0;
    return rc;
}

// The same on CTA pairs with 256 x 512 tiles: a quarter less traffic from L2 into shared memory per FLOP, which is
// what counts once the kernel runs against the power limit.
int slime_grouped_gemm_bf16_wide(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                 int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                 const void* row_info, const unsigned long long* scatter_bases8,
                                 unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                                 const float* row_scale, void* status, void* stream)
{
    g_on_pairs   = 2;
    const int rc = grouped_gemm_impl(A, B, C, group_offsets, num_groups, M_cap, N, K, lda, ldb, ldc, epilogue, row_info, scatter_bases8,
                                     scatter_row_bytes, scatter_slots, row_scale, nullptr, 0, nullptr, status, stream);
    g_on_pairs   = 0;
    return rc;
}

// The grouped GEMM whose groups become readable while it runs: before the first tile of group g is loaded, the
// producer waits (bounded) until group_ready[g] >= step, where step is group_ready_target or, if group_ready_epoch
// is not null, the value stored there when the kernel starts. Whoever fills the rows (the streamed expert-parallel
// receive) runs beside this kernel and must have been launched before it.
int slime_grouped_gemm_bf16_gated(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                  int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                  const void* group_ready, unsigned long long group_ready_target,
                                  const void* group_ready_epoch, void* status, void* stream)
{
    return slime_grouped_gemm_bf16_gated_traced(A, B, C, group_offsets, num_groups, M_cap, N, K, lda, ldb, ldc, epilogue, group_ready,
                                                group_ready_target, group_ready_epoch, nullptr, nullptr, status, stream);
}

// The same with a trace and a dynamic tile scheduler: group_trace (u64 [2 * num_groups], device memory, may be null)
// receives, per group, when CTA 0's producer began to wait for it and when it was ready (globaltimer ns); tile_counter
// (u32 [2], zero before the first launch, may be null) makes the CTAs take tiles from a shared counter, so that a CTA
// which shares its SM with the kernel that fills the groups, or starts late, takes fewer tiles.
int slime_grouped_gemm_bf16_gated_traced(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                         int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                         const void* group_ready, unsigned long long group_ready_target,
                                         const void* group_ready_epoch, void* group_trace, void* tile_counter, void* status,
                                         void* stream)
{
    if (group_ready == nullptr) return fail("gated grouped gemm: group_ready is null");
    if (epilogue == kEpiScatterRows) return fail("gated grouped gemm: the scatter epilogue is not offered in this form");
    g_group_trace  = static_cast<unsigned long long*>(group_trace);
    g_tile_counter = static_cast<unsigned int*>(tile_counter);
    const int rc = grouped_gemm_impl(A, B, C, group_offsets, num_groups, M_cap, N, K, lda, ldb, ldc, epilogue, nullptr, nullptr, 0, 0,
                                     nullptr, static_cast<const unsigned long long*>(group_ready), group_ready_target,
                                     static_cast<const unsigned long long*>(group_ready_epoch), status, stream);
    g_group_trace  = nullptr;
    g_tile_counter = nullptr;
    return rc;
}

static int grouped_gemm_impl(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                            int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                            const void* row_info, const unsigned long long* scatter_bases8,
                            unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                            const float* row_scale, const unsigned long long* group_ready,
                            unsigned long long group_ready_target, const unsigned long long* group_ready_epoch,
                            void* status, void* stream)
{
    if (check_common(M_cap, N, K, lda, ldb)) return -1;
    if (num_groups <= 0 || group_offsets == nullptr) return fail("grouped gemm: need group offsets");
    Args a{};
    a.group_ready        = group_ready;
    a.group_ready_target = group_ready_target;
    a.group_ready_epoch  = group_ready_epoch;
    a.group_trace        = g_group_trace;
    a.tile_counter       = g_tile_counter;
    a.w_prefetch         = g_w_prefetch;
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
            return g_on_pairs == 3 ? launch_pair_swapped<kEpiStore>(A, B, a, lda, ldb, s)
                   : g_on_pairs == 2 ? launch_pair_wide<kEpiStore>(A, B, a, lda, ldb, s)
                   : g_on_pairs ? launch_pair_grouped<kEpiStore>(A, B, a, lda, ldb, s) : launch<kEpiStore>(A, B, a, lda, ldb, s);
        case kEpiSwiGLU:
            if (N % 32 != 0) return fail("grouped gemm: SwiGLU needs N to be a multiple of 32");
            a.rowsB = 2 * N;
            return g_on_pairs == 3 ? launch_pair_swapped<kEpiSwiGLU>(A, B, a, lda, ldb, s)
                   : g_on_pairs == 2 ? launch_pair_wide<kEpiSwiGLU>(A, B, a, lda, ldb, s)
                   : g_on_pairs ? launch_pair_grouped<kEpiSwiGLU>(A, B, a, lda, ldb, s) : launch<kEpiSwiGLU>(A, B, a, lda, ldb, s);
        case kEpiScatterRows:
            if (row_info == nullptr || scatter_bases8 == nullptr) return fail("grouped gemm: scatter epilogue needs row_info and bases");
            if (scatter_row_bytes % 16 != 0) return fail("grouped gemm: scatter rows must be 16-byte aligned");
            a.rowsB     = N;
            a.row_info  = static_cast<const unsigned long long*>(row_info);
            a.row_scale = row_scale;
            for (int i = 0; i < 8; ++i) a.scatter_base[i] = scatter_bases8[i];
            a.scatter_row_bytes = scatter_row_bytes;
            a.scatter_slots     = scatter_slots;
            return g_on_pairs == 3 ? launch_pair_swapped<kEpiScatterRows>(A, B, a, lda, ldb, s)
                   : g_on_pairs == 2 ? launch_pair_wide<kEpiScatterRows>(A, B, a, lda, ldb, s)
                   : g_on_pairs ? launch_pair_grouped<kEpiScatterRows>(A, B, a, lda, ldb, s)
                                : launch<kEpiScatterRows>(A, B, a, lda, ldb, s);
        default:
            return fail("grouped gemm: unknown epilogue %d", epilogue);
    }
}

// The grouped GEMM with A as received from the dispatch: e4m3 rows Aq [M_cap, K] (lda in bytes) and their 1x128 scales
// a_scale [M_cap, K/128]. epilogue: kEpiStore or kEpiSwiGLU.
int slime_grouped_gemm_fp8a(const void* Aq, const float* a_scale, const void* B, void* C, const int* group_offsets, int num_groups,
                            int M_cap, int N, int K, long long lda_bytes, long long ldb, long long ldc, int epilogue, void* status,
                            void* stream)
{
    if (check_common(M_cap, N, K, 8, ldb)) return -1;
    if (K % 128 != 0 || lda_bytes % 16 != 0) return fail("fp8-A grouped gemm: K must be a multiple of 128 and lda of 16 bytes");
    if (num_groups <= 0 || group_offsets == nullptr || a_scale == nullptr) return fail("fp8-A grouped gemm: need group offsets and scales");
    Args a{};
    a.M_total       = M_cap;
    a.N             = N;
    a.K             = K;
    a.num_groups    = num_groups;
    a.group_offsets = group_offsets;
    a.C             = static_cast<__nv_bfloat16*>(C);
    a.ldc           = ldc;
    a.a_scale       = a_scale;
    a.status        = static_cast<KernelStatus*>(status);
    cudaStream_t s  = static_cast<cudaStream_t>(stream);
    if (epilogue == kEpiStore) {
        a.rowsB = N;
        return launch_a8<kEpiStore>(Aq, B, a, lda_bytes, ldb, s);
    }
    if (epilogue == kEpiSwiGLU) {
        if (N % (kBN / 2) != 0) return fail("fp8-A grouped gemm: SwiGLU needs N to be a multiple of %d", kBN / 2);
        a.rowsB = 2 * N;
        return launch_a8<kEpiSwiGLU>(Aq, B, a, lda_bytes, ldb, s);
    }
    return fail("fp8-A grouped gemm: unknown epilogue %d", epilogue);
}

}  // extern "C"
