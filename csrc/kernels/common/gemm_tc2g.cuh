// The grouped expert GEMM on CTA PAIRS (tcgen05 cta_group::2): the pair mechanics of gemm_tc2.cuh (every CTA
// loads its 128 rows of A and its half of the B rows, one thread of the leader issues M = 256 MMAs, commits with a
// CTA mask) with the row groups and the epilogues of gemm_tc.cuh (store, SwiGLU, scatter rows).
//
// Why: a single CTA with a 128 x 256 tile has to pull 48 KB from L2 for every 64-deep K block, which takes longer
// than the four MMAs of that block (the tensor pipe of the single-CTA kernel sits at ~71 %); in a pair each CTA pulls
// 32 KB for the same MMA time. The price is 256-row tiles: the last tile of a group computes up to 255 rows that
// are never stored, so pairs pay off where groups are large (many ranks: ~1000 rows per expert) and the single-CTA
// kernel stays the choice for small groups.
//
// Tiles of a group: row tiles of 256 (m fastest), n tiles of BN. For SwiGLU the leader loads the gate rows of the
// weight and the peer the up rows, so that accumulator columns [0, BN/2) are gate and [BN/2, BN) up in both CTAs'
// tensor memory, exactly the layout the single-CTA epilogue expects.
#pragma once

#include "gemm_tc2.cuh"

namespace slime {
namespace gemm {

struct PairGTile {
    int group;
    int row0;     // first of the 256 rows of the tile
    int row_end;  // one past the last valid row of the group
    int nt;
};

struct PairGroupWalker {
    const Args& a;
    int         ntiles_n, t, step, g, cum, g_begin, g_end, g_mtiles;
    __device__ PairGroupWalker(const Args& args, int bn_out, int cluster, int n_clusters): a(args)
    {
        ntiles_n = (a.N + bn_out - 1) / bn_out;
        t        = cluster;
        step     = n_clusters;
        g        = -1;
        cum      = 0;
        g_begin = g_end = g_mtiles = 0;
        advance_group();
    }
    __device__ void advance_group()
    {
        ++g;
        if (g < a.num_groups) {
            g_begin = a.group_offsets ? a.group_offsets[g] : 0;
            g_end   = a.group_offsets ? a.group_offsets[g + 1] : a.M_total;
            if (g_end > a.M_total) g_end = a.M_total;
            if (g_begin > g_end) g_begin = g_end;
            g_mtiles = (g_end - g_begin + kPairBM - 1) / kPairBM;
        }
    }
    __device__ bool next(PairGTile& c)
    {
        while (g < a.num_groups) {
            const int tiles_g = g_mtiles * ntiles_n;
            if (t < cum + tiles_g) {
                const int local = t - cum;
                c.group   = g;
                c.row0    = g_begin + (local % g_mtiles) * kPairBM;
                c.row_end = g_end;
                c.nt      = local / g_mtiles;
                t += step;
                return true;
            }
            cum += tiles_g;
            advance_group();
        }
        return false;
    }
};

template<int BN, int STAGES, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_pair_grouped_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Args args)
{
    using S = SmemPair<BN, STAGES, false>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    uint8_t*  epi_smem   = smem + STAGES * S::kStageBytes;
    uint64_t* full_bar   = reinterpret_cast<uint64_t*>(epi_smem + S::kEpiBytes);  // used in the leader only
    uint64_t* empty_bar  = full_bar + STAGES;                                     // one set per CTA
    uint64_t* tfull_bar  = empty_bar + STAGES;                                    // [2] per CTA
    uint64_t* tempty_bar = tfull_bar + 2;                                         // [2] used in the leader only
    uint32_t* tmem_slot  = reinterpret_cast<uint32_t*>(tempty_bar + 2 + kAgMaxBufs);
    volatile uint32_t* fail_slot = tmem_slot + 1;

    const int          warp    = threadIdx.x >> 5;
    const int          lane    = threadIdx.x & 31;
    const uint32_t     crank   = cluster_ctarank();  // 0 = leader
    const int          cluster = blockIdx.x >> 1;
    const int          n_clusters = gridDim.x >> 1;
    const int          kblocks = (args.K + kBK - 1) / kBK;
    KernelStatus*      st      = args.status;
    const unsigned long long lim = args.wait_ns ? args.wait_ns : kDefaultWaitNs;
    constexpr int      kAccStride = BN <= 128 ? 128 : 256;
    constexpr int      kTmemCols  = 2 * kAccStride;
    constexpr int      kBNOut     = (EPI == kEpiSwiGLU) ? BN / 2 : BN;
    static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "tile width");

    if (threadIdx.x == 0) {
        *fail_slot = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);   // the leader's producer arrives once and expects the bytes of both CTAs
            mbar_init(&empty_bar[s], 1);  // one commit
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tfull_bar[s], 1);
            mbar_init(&tempty_bar[s], 256);  // the epilogue threads of both CTAs
        }
        fence_mbar_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything is sent to them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer (both CTAs) ------------------------------
        if (lane == 0) {
            PairGroupWalker walk(args, kBNOut, cluster, n_clusters);
            PairGTile       tc;
            int             stage = 0;
            uint32_t        phase = 0;
            bool            ok    = true;
            while (ok && walk.next(tc)) {
                const int arow = tc.row0 + static_cast<int>(crank) * kBM;
                int       yb;
                if (EPI == kEpiSwiGLU)  // leader: gate rows of this n tile; peer: the matching up rows
                    yb = tc.group * args.rowsB + (crank == 0 ? 0 : args.N) + tc.nt * (BN / 2);
                else
                    yb = tc.group * args.rowsB + tc.nt * BN + static_cast<int>(crank) * (BN / 2);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, st, 1, stage, lim)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * S::kStageBytes;
                    uint8_t* sb = sa + S::kABytes;
                    if (crank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * S::kStageBytes);
                    const uint32_t leader_full = mapa_u32(&full_bar[stage], 0);
                    tma_load_2d_pair(sa, &tmA, leader_full, kb * kBK, arow);
                    tma_load_2d_pair(sb, &tmB, leader_full, kb * kBK, yb);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) *fail_slot = 1;
        }
    }
    else if (warp == 1) {
        // ------------------------------ MMA issuer (leader only) ------------------------------
        if (lane == 0 && crank == 0) {
            PairGroupWalker walk(args, kBNOut, cluster, n_clusters);
            PairGTile       tc;
            int             stage = 0;
            uint32_t        phase = 0;
            int             acc = 0;
            uint32_t        acc_phase = 0;
            bool            ok = true;
            constexpr uint32_t idesc = make_idesc(kFmtBF16, kFmtBF16, kPairBM, BN);
            while (ok && walk.next(tc)) {
                if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, st, 2, acc, lim)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc * kAccStride;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, st, 3, stage, lim)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
                    const uint32_t sb = sa + S::kABytes;
                    const uint64_t da = make_kmajor_sw128_desc(sa);
                    const uint64_t db = make_kmajor_sw128_desc(sb);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) umma_f16_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    umma_commit_pair(&empty_bar[stage], 3);  // frees the stage in both CTAs
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit_pair(&tfull_bar[acc], 3);  // the accumulator halves of both CTAs are complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
            if (!ok) *fail_slot = 1;
        }
    }
    else {
        // ------------------------------ epilogue (both CTAs, own TMEM rows) ------------------------------
        const int       quad = warp & 3;
        PairGroupWalker walk(args, kBNOut, cluster, n_clusters);
        PairGTile       tc;
        int             acc = 0;
        uint32_t        acc_phase = 0;
        const uint32_t  leader_tempty[2] = {mapa_u32(&tempty_bar[0], 0), mapa_u32(&tempty_bar[1], 0)};
        while (walk.next(tc)) {
            if (!mbar_wait(&tfull_bar[acc], acc_phase, st, 4, acc, lim)) {
                *fail_slot = 1;
                break;
            }
            tc_fence_after_sync();
            const int      row   = tc.row0 + static_cast<int>(crank) * kBM + quad * 32 + lane;
            const bool     valid = row < tc.row_end;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kAccStride;
            const int      col0  = tc.nt * kBNOut;
            unsigned long long drow = 0;
            float              scale = 1.0f;
            bool               do_store = valid;
            if (EPI == kEpiScatterRows) {
                const unsigned long long inf    = valid ? args.row_info[row] : ~0ull;
                const unsigned int       region = static_cast<unsigned int>(inf >> 48);
                const unsigned long long slot   = inf & 0xffffffffffffull;
                const unsigned long long base   = region < 8 ? args.scatter_base[region] : 0ull;
                do_store                        = valid && base != 0ull && slot < args.scatter_slots;
                drow = base + slot * args.scatter_row_bytes + static_cast<unsigned long long>(col0) * 2;
                if (do_store && args.row_scale) scale = args.row_scale[row];
            }
            else {
                drow = reinterpret_cast<unsigned long long>(args.C + static_cast<long long>(row) * args.ldc + col0);
            }
            uint8_t* my_slot = epi_smem + (quad * 32 + lane) * kEpiRowPitch;
            const uint8_t* warp_slots = epi_smem + quad * 32 * kEpiRowPitch;
#pragma unroll 1
            for (int c = 0; c < kBNOut; c += 64) {
                uint32_t o[32];
                if (EPI == kEpiSwiGLU) {
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb) {
                        uint32_t g[32], u[32];
                        tmem_ld_32x32b_x32(taddr + c + hb * 32, g);
                        tmem_ld_32x32b_x32(taddr + BN / 2 + c + hb * 32, u);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float h0 = silu(__uint_as_float(g[2 * i])) * __uint_as_float(u[2 * i]);
                            const float h1 = silu(__uint_as_float(g[2 * i + 1])) * __uint_as_float(u[2 * i + 1]);
                            o[hb * 16 + i] = pack_bf16(h0, h1);
                        }
                    }
                }
                else {
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb) {
                        uint32_t v[32];
                        tmem_ld_32x32b_x32(taddr + c + hb * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            o[hb * 16 + i] = pack_bf16(__uint_as_float(v[2 * i]) * scale, __uint_as_float(v[2 * i + 1]) * scale);
                    }
                }
                int cols = args.N - (col0 + c);
                if (cols > 64) cols = 64;
                if (cols > kBNOut - c) cols = kBNOut - c;
                epi_store_piece(my_slot, warp_slots, o, drow + static_cast<unsigned long long>(c) * 2, do_store, cols, lane);
            }
            tc_fence_before_sync();
            if (crank == 0)
                mbar_arrive(&tempty_bar[acc]);
            else
                mbar_arrive_cluster(leader_tempty[acc]);
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
    }

    // teardown: both CTAs meet (no CTA may leave while its peer still reads its shared memory or signals its
    // barriers), then the allocating warps free TMEM
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        if (*fail_slot != 0) {
            const unsigned long long t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

}  // namespace gemm
}  // namespace slime
