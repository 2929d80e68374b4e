// The bf16 GEMM main loop on CTA PAIRS (tcgen05 cta_group::2): a cluster of two CTAs on two SMs works
// on one 256 x BN output tile.
//
//   * every CTA loads ITS 128 rows of A and ITS half of the B rows (BN/2) of each 64-wide K block, so a
//     pair reads each B tile once instead of twice and a stage is 32 KB per CTA: the ring is 6 deep
//     where the single-CTA kernel has room for 4, which covers more load latency, and the traffic
//     between L2 and the SMs drops by a third;
//   * the loads of both CTAs complete on the LEADER's (even CTA's) "full" barrier; one thread of the
//     leader issues tcgen05.mma.cta_group::2 (M = 256), which reads A and B from both CTAs' shared
//     memory and accumulates into both CTAs' TMEM (128 rows each);
//   * tcgen05.commit with a CTA mask releases the stage ("empty") and publishes the accumulator
//     ("tfull") in both CTAs at once; the epilogue warps of both CTAs drain their own TMEM and arrive
//     on the leader's "tempty" barrier (the peer's arrivals are remote).
//
// This file: one group (plain GEMM and all-gather -> GEMM). The grouped forms on pairs are gemm_tc2g.cuh
// (256 x 256 tiles per group), gemm_tc2w.cuh (256 x 512 tiles) and gemm_tc2s.cuh (operands swapped). Same Args,
// same bounded waits, same status page as gemm_tc.cuh; the all-gather roles (gating on arrival counters,
// shard-major tile order, the push warp) carry over.
#pragma once

#include "gemm_tc.cuh"

namespace slime {
namespace gemm {

constexpr int kPairBM = 256;

template<int BN, int STAGES, bool AG = false>
struct SmemPair {
    static constexpr int kABytes     = kBM * kBK * 2;         // this CTA's 128 rows
    static constexpr int kBBytes     = (BN / 2) * kBK * 2;    // this CTA's half of the B rows
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarBytes   = (2 * STAGES + 4 + kAgMaxBufs) * 8 + 16;
    static constexpr int kEpiBytes   = 128 * kEpiRowPitch;
    static constexpr int kBase       = STAGES * kStageBytes + kEpiBytes + kBarBytes + 1024;
    static constexpr int kAgBufs = !AG ? 0 : ((kSmemLimit - kBase - 128) / kAgChunkBytes > kAgMaxBufs ? kAgMaxBufs : (kSmemLimit - kBase - 128) / kAgChunkBytes);
    static constexpr int kTotal  = kBase + (AG ? kAgBufs * kAgChunkBytes + 128 : 0);
    static_assert(kStageBytes % 1024 == 0, "stage alignment for the 128-byte swizzle");
    static_assert(kTotal <= kSmemLimit, "shared memory budget");
    static_assert(!AG || kAgBufs >= 2, "no room for the push buffers");
};

struct PairTile {
    int row0;  // first of the 256 rows of the tile
    int nt;
};

// Tiles t = cluster, cluster + n_clusters, ... ; shard-major for the all-gather form, else in bands of tile columns
// whose B rows (at most ~40 MB) stay in L2 while A streams past once per band; inside a band the column runs fastest.
struct PairWalker {
    const Args& a;
    int         mtiles, ntiles, total, t, step, band;
    __device__ PairWalker(const Args& args, int bn, int cluster, int n_clusters): a(args)
    {
        mtiles = (a.M_total + kPairBM - 1) / kPairBM;
        ntiles = (a.N + bn - 1) / bn;
        total  = mtiles * ntiles;
        t      = cluster;
        step   = n_clusters;
        const long long per_col = static_cast<long long>(bn) * a.K * 2;
        const long long b       = (40ll << 20) / (per_col > 0 ? per_col : 1);
        band                    = b < 1 ? 1 : (b > ntiles ? ntiles : static_cast<int>(b));
    }
    __device__ bool next(PairTile& c)
    {
        if (t >= total) return false;
        int mt, nt;
        if (a.ag_shard_order) {
            const int per       = a.ag_rows / kPairBM;
            const int per_shard = per * ntiles;
            const int j         = t / per_shard;
            const int rem       = t - j * per_shard;
            const int shard     = ((a.ag_rank - j) % a.ag_world + a.ag_world) % a.ag_world;
            nt                  = rem / per;
            mt                  = shard * per + rem % per;
        }
        else {
            const int per_band = mtiles * band;
            const int b        = t / per_band;
            const int r        = t - b * per_band;
            const int width    = (b + 1) * band <= ntiles ? band : ntiles - b * band;  // the last band may be narrower
            mt                 = r / width;
            nt                 = b * band + r % width;
        }
        c.row0 = mt * kPairBM;
        c.nt   = nt;
        t += step;
        return true;
    }
};

template<int BN, int STAGES, bool AG = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads + (AG ? kAgThreads : 0), 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmAL, const Args args)
{
    using S = SmemPair<BN, STAGES, AG>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    uint8_t*  epi_smem   = smem + STAGES * S::kStageBytes;
    uint64_t* full_bar   = reinterpret_cast<uint64_t*>(epi_smem + S::kEpiBytes);  // used in the leader only
    uint64_t* empty_bar  = full_bar + STAGES;                                     // one set per CTA
    uint64_t* tfull_bar  = empty_bar + STAGES;                                    // [2] per CTA
    uint64_t* tempty_bar = tfull_bar + 2;                                         // [2] used in the leader only
    uint64_t* ag_bar     = tempty_bar + 2;
    uint32_t* tmem_slot  = reinterpret_cast<uint32_t*>(ag_bar + kAgMaxBufs);
    volatile uint32_t* fail_slot = tmem_slot + 1;
    uint8_t*  ag_bufs    = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(epi_smem + S::kEpiBytes + S::kBarBytes) + 127) & ~uintptr_t(127));

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
    static_assert(BN % 32 == 0 && BN >= 64 && BN <= 256, "tile width");

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
        if (AG)
            for (int s = 0; s < kAgMaxBufs; ++s) mbar_init(&ag_bar[s], 1);
        fence_mbar_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if (AG) tma_prefetch_desc(&tmAL);
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
            PairWalker walk(args, BN, cluster, n_clusters);
            PairTile   tc;
            int        stage = 0;
            uint32_t   phase = 0;
            bool       ok    = true;
            while (ok && walk.next(tc)) {
                const int          my_row0 = tc.row0 + static_cast<int>(crank) * kBM;
                const CUtensorMap* mapA = &tmA;
                int                arow = my_row0;
                bool               gate = args.a_ready != nullptr && my_row0 < args.M_total;
                if (AG && args.ag_local_direct && my_row0 / args.ag_rows == args.ag_rank) {
                    mapA = &tmAL;
                    arow = my_row0 - args.ag_rank * args.ag_rows;
                    gate = false;
                }
                if (gate) {
                    const int f = my_row0 / args.a_ready_rows;  // a_ready_rows == 128: one counter per CTA half
                    ok = wait_flag_ge(args.a_ready + f, args.a_ready_target, st, 10, f, lim);
                    if (!ok) break;
                    fence_proxy_async();
                }
                const int yb = tc.nt * BN + static_cast<int>(crank) * (BN / 2);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, st, 1, stage, lim)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * S::kStageBytes;
                    uint8_t* sb = sa + S::kABytes;
                    if (crank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * S::kStageBytes);
                    const uint32_t leader_full = mapa_u32(&full_bar[stage], 0);
                    tma_load_2d_pair(sa, mapA, leader_full, kb * kBK, arow);
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
            PairWalker walk(args, BN, cluster, n_clusters);
            PairTile   tc;
            int        stage = 0;
            uint32_t   phase = 0;
            int        acc = 0;
            uint32_t   acc_phase = 0;
            bool       ok = true;
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
    else if (AG && warp >= 6) {
        // ------------------------------ all-gather push ------------------------------
        if (args.ag_src != nullptr && lane == 0) {
            if (!ag_push_bulk(args, ag_bufs, ag_bar, S::kAgBufs, blockIdx.x, gridDim.x, st, lim)) *fail_slot = 1;
        }
    }
    else {
        // ------------------------------ epilogue (both CTAs, own TMEM rows) ------------------------------
        const int      quad = warp & 3;
        PairWalker     walk(args, BN, cluster, n_clusters);
        PairTile       tc;
        int            acc = 0;
        uint32_t       acc_phase = 0;
        const uint32_t leader_tempty[2] = {mapa_u32(&tempty_bar[0], 0), mapa_u32(&tempty_bar[1], 0)};
        while (walk.next(tc)) {
            if (!mbar_wait(&tfull_bar[acc], acc_phase, st, 4, acc, lim)) {
                *fail_slot = 1;
                break;
            }
            tc_fence_after_sync();
            const int      row   = tc.row0 + static_cast<int>(crank) * kBM + quad * 32 + lane;
            const bool     valid = row < args.M_total;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kAccStride;
            const int      col0  = tc.nt * BN;
            const unsigned long long drow = reinterpret_cast<unsigned long long>(args.C + static_cast<long long>(row) * args.ldc + col0);
            uint8_t* my_slot = epi_smem + (quad * 32 + lane) * kEpiRowPitch;
            const uint8_t* warp_slots = epi_smem + quad * 32 * kEpiRowPitch;
#pragma unroll 1
            for (int c = 0; c < BN; c += 64) {
                uint32_t o[32];
#pragma unroll
                for (int hb = 0; hb < 2; ++hb) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c + hb * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[hb * 16 + i] = pack_bf16(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                }
                int cols = args.N - (col0 + c);
                if (cols > 64) cols = 64;
                if (cols > BN - c) cols = BN - c;
                epi_store_piece(my_slot, warp_slots, o, drow + static_cast<unsigned long long>(c) * 2, valid, cols, lane);
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
