// The bf16 GEMM on CTA pairs with WIDE tiles: one pair works on 256 rows x (2 x BN) columns, as two accumulator
// blocks of BN columns that share the A tile. Plain GEMMs and grouped (expert) GEMMs, every epilogue.
//
// Why: on this part a large GEMM runs against the board's power limit, not against the tensor pipe. The 256 x 256
// pair kernel keeps the tensor pipe 97 % busy and still loses to the vendor library, because it draws more power
// per FLOP and the clock drops (990 MHz against 1200 MHz in a seconds-long loop of 8192^3). What differs is data
// movement: per 64-deep K block a pair with a 256 x 256 tile pulls 64 KB from L2 into shared memory, a pair with
// a 256 x 512 tile pulls 96 KB for twice the FLOPs, a quarter less per FLOP (and a quarter fewer shared-memory
// writes). The second lever is the order of the tiles of a one-group GEMM: bands of a few tile columns, so that
// the B rows of a band stay in L2 while A streams past once per band (the m-fastest order re-read A from HBM in
// every wave: 2.3 GB of DRAM reads for 8192^3 where 0.4 GB are needed).
//
// Price: the two blocks fill all 512 tensor-memory columns, so the accumulators are not double buffered and the
// drain of a tile is exposed. To keep it short there are eight epilogue warps, four per block: both blocks drain at
// once, a warp first pulls its whole block into registers (packed to bf16) and hands the block back before it
// stores anything, so what the tensor pipe waits for is the tensor-memory reads alone; the stores run under the
// next tile's main loop.
//
// Shared memory per stage and CTA: A 128 x 64 (16 KB), then this CTA's half of the B rows of block 0 and of block 1
// (BN/2 x 64 each). Four stages.
#pragma once

#include "gemm_tc2g.cuh"

namespace slime {
namespace gemm {

template<int BN, int STAGES>
struct SmemWide {
    static constexpr int kABytes     = kBM * kBK * 2;
    static constexpr int kBHalfBytes = (BN / 2) * kBK * 2;  // one block's half
    static constexpr int kStageBytes = kABytes + 2 * kBHalfBytes;
    static constexpr int kBarBytes   = (2 * STAGES + 4 + kAgMaxBufs) * 8 + 16;
    static constexpr int kEpiBytes   = 256 * kEpiRowPitch;  // eight epilogue warps
    static constexpr int kTotal      = STAGES * kStageBytes + kEpiBytes + kBarBytes + 1024;
    static_assert(kBHalfBytes % 1024 == 0 && kStageBytes % 1024 == 0, "operand alignment for the 128-byte swizzle");
    static_assert(kTotal <= kSmemLimit, "shared memory budget");
};

constexpr int kWideThreads = 64 + 256;  // producer warp, MMA warp, four epilogue warps per accumulator block

struct WideTile {
    int group;
    int row0;     // first of the 256 rows
    int row_end;  // one past the last valid row of the group
    int nt;       // tile column (2 x BN wide)
};

// Tiles t = cluster, cluster + n_clusters, ... One group without offsets: bands of `band` tile columns, inside a band
// the tile column runs fastest. Several groups: group by group, rows fastest (the tiles of a wave share weight rows).
struct WideWalker {
    const Args& a;
    int         ntiles_n, t, step, g, cum, g_begin, g_end, g_mtiles, band;
    bool        plain;
    __device__ WideWalker(const Args& args, int tile_out, int cluster, int n_clusters): a(args)
    {
        ntiles_n = (a.N + tile_out - 1) / tile_out;
        t        = cluster;
        step     = n_clusters;
        plain    = a.num_groups == 1 && a.group_offsets == nullptr;
        g        = -1;
        cum      = 0;
        g_begin = g_end = g_mtiles = 0;
        // B rows of a band: at most ~40 MB, so that they stay in L2 next to the A rows that stream past
        const long long per_col = static_cast<long long>(tile_out) * a.K * 2;
        long long       b       = (40ll << 20) / (per_col > 0 ? per_col : 1);
        band                    = b < 1 ? 1 : (b > ntiles_n ? ntiles_n : static_cast<int>(b));
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
    __device__ bool next(WideTile& c)
    {
        if (plain) {
            if (t >= g_mtiles * ntiles_n) return false;
            const int per_band = g_mtiles * band;
            const int b        = t / per_band;
            const int r        = t - b * per_band;
            const int width    = (b + 1) * band <= ntiles_n ? band : ntiles_n - b * band;  // the last band may be narrower
            c.group   = 0;
            c.row0    = (r / width) * kPairBM;
            c.row_end = g_end;
            c.nt      = b * band + r % width;
            t += step;
            return true;
        }
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
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kWideThreads, 1)
gemm_bf16_pair_wide_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Args args)
{
    using S = SmemWide<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    uint8_t*  epi_smem   = smem + STAGES * S::kStageBytes;
    uint64_t* full_bar   = reinterpret_cast<uint64_t*>(epi_smem + S::kEpiBytes);  // used in the leader only
    uint64_t* empty_bar  = full_bar + STAGES;                                     // one set per CTA
    uint64_t* tfull_bar  = empty_bar + STAGES;                                    // [2]: one per accumulator block, per CTA
    uint64_t* tempty_bar = tfull_bar + 2;                                         // [2]: used in the leader only
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
    constexpr int      kAccStride = 256;
    constexpr int      kTmemCols  = 512;
    constexpr int      kBNOut     = (EPI == kEpiSwiGLU) ? BN / 2 : BN;  // output columns of one block
    constexpr int      kTileOut   = 2 * kBNOut;
    static_assert(BN % 64 == 0 && BN >= 128 && BN <= 256, "block width");

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
            WideWalker walk(args, kTileOut, cluster, n_clusters);
            WideTile   tc;
            int        stage = 0;
            uint32_t   phase = 0;
            bool       ok    = true;
            while (ok && walk.next(tc)) {
                const int arow = tc.row0 + static_cast<int>(crank) * kBM;
                int       yb[2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    if (EPI == kEpiSwiGLU)  // leader: gate rows of block j; peer: the matching up rows
                        yb[j] = tc.group * args.rowsB + (crank == 0 ? 0 : args.N) + tc.nt * kTileOut + j * kBNOut;
                    else
                        yb[j] = tc.group * args.rowsB + tc.nt * kTileOut + j * BN + static_cast<int>(crank) * (BN / 2);
                }
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
                    tma_load_2d_pair(sb, &tmB, leader_full, kb * kBK, yb[0]);
                    tma_load_2d_pair(sb + S::kBHalfBytes, &tmB, leader_full, kb * kBK, yb[1]);
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
            WideWalker walk(args, kTileOut, cluster, n_clusters);
            WideTile   tc;
            int        stage = 0;
            uint32_t   phase = 0;
            uint32_t   tile_phase = 0;
            bool       ok = true;
            constexpr uint32_t idesc = make_idesc(kFmtBF16, kFmtBF16, kPairBM, BN);
            while (ok && walk.next(tc)) {
                const bool two = tc.nt * kTileOut + kBNOut < args.N;  // block 1 holds columns of the output
                for (int kb = 0; kb < kblocks && ok; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, st, 3, stage, lim)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
                    const uint64_t da = make_kmajor_sw128_desc(sa);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        if (kb == 0) {  // the epilogue has drained this block of the previous tile
                            if (!mbar_wait(&tempty_bar[j], tile_phase ^ 1, st, 2, j, lim)) {
                                ok = false;
                                break;
                            }
                            tc_fence_after_sync();
                        }
                        if (j == 0 || two) {
                            const uint64_t db = make_kmajor_sw128_desc(sa + S::kABytes + j * S::kBHalfBytes);
#pragma unroll
                            for (int k = 0; k < kBK / 16; ++k)
                                umma_f16_pair(tmem_base + j * kAccStride, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                        }
                        if (kb == kblocks - 1 && j == 0) umma_commit_pair(&tfull_bar[0], 3);  // block 0 is complete
                    }
                    if (!ok) break;
                    umma_commit_pair(&empty_bar[stage], 3);  // frees the stage in both CTAs
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit_pair(&tfull_bar[1], 3);
                tile_phase ^= 1;
            }
            if (!ok) *fail_slot = 1;
        }
    }
    else {
        // ------------------------------ epilogue (both CTAs, own TMEM rows) ------------------------------
        const int      quad = warp & 3;          // the TMEM lanes a warp may read: 32 * (warp % 4)
        const int      j    = warp >= 6 ? 1 : 0;  // warps 2..5 drain block 0, warps 6..9 block 1
        WideWalker     walk(args, kTileOut, cluster, n_clusters);
        WideTile       tc;
        uint32_t       tile_phase = 0;
        const uint32_t leader_tempty = mapa_u32(&tempty_bar[j], 0);
        uint8_t*       my_slot    = epi_smem + ((j * 4 + quad) * 32 + lane) * kEpiRowPitch;
        const uint8_t* warp_slots = epi_smem + (j * 4 + quad) * 32 * kEpiRowPitch;
        while (walk.next(tc)) {
            const int  row   = tc.row0 + static_cast<int>(crank) * kBM + quad * 32 + lane;
            const bool valid = row < tc.row_end;
            const int  col0  = tc.nt * kTileOut + j * kBNOut;
            unsigned long long drow = 0;
            float              scale = 1.0f;
            bool               do_store = valid && col0 < args.N;
            if (EPI == kEpiScatterRows) {
                const unsigned long long info   = valid ? args.row_info[row] : ~0ull;
                const unsigned int       region = static_cast<unsigned int>(info >> 48);
                const unsigned long long slot   = info & 0xffffffffffffull;
                const unsigned long long base   = region < 8 ? args.scatter_base[region] : 0ull;
                do_store                        = do_store && base != 0ull && slot < args.scatter_slots;
                drow = base + slot * args.scatter_row_bytes + static_cast<unsigned long long>(col0) * 2;
                if (do_store && args.row_scale) scale = args.row_scale[row];
            }
            else {
                drow = reinterpret_cast<unsigned long long>(args.C + static_cast<long long>(row) * args.ldc + col0);
            }
            if (!mbar_wait_relaxed(&tfull_bar[j], tile_phase, st, 4, j, lim)) {
                *fail_slot = 1;
                break;
            }
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + j * kAccStride;
            // Drain first, store afterwards: the whole block goes to registers as packed bf16 (kBNOut / 2 words), the
            // block is handed back to the MMA warp, and only then do the rows leave through shared memory, under the
            // next tile's main loop.
            uint32_t packed[kBNOut / 2];
            if (col0 < args.N) {
#pragma unroll
                for (int c = 0; c < kBNOut; c += 64) {
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
                                packed[c / 2 + hb * 16 + i] = pack_bf16(h0, h1);
                            }
                        }
                    }
                    else {
                        uint32_t v0[32], v1[32];  // both halves in flight before the one wait
                        tmem_ld_32x32b_x32(taddr + c, v0);
                        tmem_ld_32x32b_x32(taddr + c + 32, v1);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            packed[c / 2 + i]      = pack_bf16(__uint_as_float(v0[2 * i]) * scale, __uint_as_float(v0[2 * i + 1]) * scale);
                            packed[c / 2 + 16 + i] = pack_bf16(__uint_as_float(v1[2 * i]) * scale, __uint_as_float(v1[2 * i + 1]) * scale);
                        }
                    }
                }
            }
            tc_fence_before_sync();
            if (crank == 0)
                mbar_arrive(&tempty_bar[j]);
            else
                mbar_arrive_cluster(leader_tempty);
            if (col0 < args.N) {
#pragma unroll
                for (int c = 0; c < kBNOut; c += 64) {
                    uint32_t o[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = packed[c / 2 + i];
                    int cols = args.N - (col0 + c);
                    if (cols > 64) cols = 64;
                    if (cols > kBNOut - c) cols = kBNOut - c;
                    epi_store_piece(my_slot, warp_slots, o, drow + static_cast<unsigned long long>(c) * 2, do_store, cols, lane);
                }
            }
            tile_phase ^= 1;
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
