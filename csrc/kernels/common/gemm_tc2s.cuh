// The grouped expert GEMM on CTA pairs with the operands SWAPPED: the weight rows are the M side of the MMA
// (tcgen05 cta_group::2, M = 256: 128 weight rows per CTA) and the tokens of a group are the N side, which may be any
// multiple of 16 up to 256.
//
// Why. With tokens on the M side a group is cut into 128- or 256-row tiles and its last tile computes up to 127 or 255
// rows that nobody reads; at 128 +- 11 tokens per expert (one GPU, 256 experts) half of the experts cost two tiles, i.e.
// two passes over their weights from L2, for one tile's worth of tokens. With tokens on the N side a group of up to 256
// tokens is ONE tile whose MMAs are exactly as wide as the group (rounded up to 16), larger groups are cut into equal
// parts, and the weight tile is read once per part. Per 64-deep K block a CTA loads 16 KB of weights and 16 KB of tokens
// (the pair's token tile is split between the two CTAs), as the 256 x 256 pair kernel does.
//
// The accumulator is transposed (tensor-memory lanes are output features, columns are tokens), so the epilogue turns
// it around in shared memory: every thread reads 32 tokens of its feature, the four epilogue warps stage a
// 32-token x 128-feature block in fp32 (two blocks, used in turn, one named barrier per block), and then write token
// rows: 256 contiguous bytes of bf16 per token and CTA. For SwiGLU a CTA's 128 weight rows are 64 gate rows and the
// matching 64 up rows, so that gate and up of one output meet in the staged block (in fp32, before any rounding).
//
// Tiles of a group: ceil(rows / 256) equal parts (rounded up to 16 tokens), part fastest, then the feature tile
// (256 weight rows per pair: 256 output columns, or 128 for SwiGLU).
//
// Measured (32 / 64 / 128 / 256 experts with 1024 / 512 / 256 / 128 rows on average, router-like sizes): level with the
// 256 x 256 pair kernel at 1024 rows per expert (gate/up 1.373 against 1.368 ms), and behind the single-CTA kernel on
// smaller groups (256 x 128: 3.34 + 1.80 ms against 2.67 + 1.38 ms) although it computes a third fewer rows and reads
// the weights from L2 once instead of 1.5 times: those launches stream weights from HBM, and 148 CTAs that each
// keep 128 KB of weight tiles in flight pull more from HBM than 74 pairs with 96 KB per CTA. The expert-parallel layer
// times this form with the others (`ExpertParallelMoE.autotune`) and has not picked it so far.
#pragma once

#include "gemm_tc2g.cuh"

namespace slime {
namespace gemm {

constexpr int kSwapTokens = 256;  // most tokens per tile (the N of the MMA)

template<int STAGES>
struct SmemSwap {
    static constexpr int kWBytes     = kBM * kBK * 2;  // this CTA's 128 weight rows
    static constexpr int kXBytes     = kBM * kBK * 2;  // this CTA's half of the token rows (a box of 128)
    static constexpr int kStageBytes = kWBytes + kXBytes;
    static constexpr int kBlockBytes = 32 * 128 * 4;   // one staged block: 32 tokens x 128 features, fp32
    static constexpr int kEpiBytes   = 2 * kBlockBytes;
    static constexpr int kBarBytes   = (2 * STAGES + 4) * 8 + 32;
    static constexpr int kTotal      = STAGES * kStageBytes + kEpiBytes + kBarBytes + 1024;
    static_assert(kTotal <= kSmemLimit, "shared memory budget");
};

struct SwapTile {
    int group;
    int tok0;     // first token row of the tile
    int tok_end;  // one past its last valid token row
    int ntok;     // N of the MMAs: the valid tokens rounded up to 16 (at least 16)
    int nt;       // feature tile
};

struct SwapWalker {
    const Args& a;
    int         ntiles_n, t, step, g, cum, g_begin, g_end, g_parts, g_part_rows;
    __device__ SwapWalker(const Args& args, int feat_out, int cluster, int n_clusters): a(args)
    {
        ntiles_n = (a.N + feat_out - 1) / feat_out;
        t        = cluster;
        step     = n_clusters;
        g        = -1;
        cum      = 0;
        g_begin = g_end = g_parts = g_part_rows = 0;
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
            const int rows = g_end - g_begin;
            g_parts        = (rows + kSwapTokens - 1) / kSwapTokens;
            g_part_rows    = g_parts ? (((rows + g_parts - 1) / g_parts + 15) & ~15) : 0;  // <= 256
        }
    }
    __device__ bool next(SwapTile& c)
    {
        while (g < a.num_groups) {
            const int tiles_g = g_parts * ntiles_n;
            if (t < cum + tiles_g) {
                const int local = t - cum;
                const int part  = local % g_parts;
                c.group   = g;
                c.tok0    = g_begin + part * g_part_rows;
                c.tok_end = c.tok0 + g_part_rows < g_end ? c.tok0 + g_part_rows : g_end;
                int valid = c.tok_end - c.tok0;
                if (valid < 0) {  // a part past the end of a very large group: nothing to store
                    valid     = 0;
                    c.tok0    = g_end;
                    c.tok_end = g_end;
                }
                c.ntok = valid <= 16 ? 16 : ((valid + 15) & ~15);
                c.nt   = local / g_parts;
                t += step;
                return true;
            }
            cum += tiles_g;
            advance_group();
        }
        return false;
    }
};

template<int STAGES, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_pair_swapped_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const Args args)
{
    using S = SmemSwap<STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    uint8_t*  epi_smem   = smem + STAGES * S::kStageBytes;
    uint64_t* full_bar   = reinterpret_cast<uint64_t*>(epi_smem + S::kEpiBytes);  // used in the leader only
    uint64_t* empty_bar  = full_bar + STAGES;                                     // one set per CTA
    uint64_t* tfull_bar  = empty_bar + STAGES;                                    // [2] per CTA
    uint64_t* tempty_bar = tfull_bar + 2;                                         // [2] used in the leader only
    uint32_t* tmem_slot  = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    volatile uint32_t* fail_slot = tmem_slot + 1;
    volatile uint32_t* epi_fail  = tmem_slot + 2;  // written by epilogue threads only, read after their named barrier

    const int          warp    = threadIdx.x >> 5;
    const int          lane    = threadIdx.x & 31;
    const uint32_t     crank   = cluster_ctarank();  // 0 = leader
    const int          cluster = blockIdx.x >> 1;
    const int          n_clusters = gridDim.x >> 1;
    const int          kblocks = (args.K + kBK - 1) / kBK;
    KernelStatus*      st      = args.status;
    const unsigned long long lim = args.wait_ns ? args.wait_ns : kDefaultWaitNs;
    constexpr int      kAccStride = kSwapTokens;
    constexpr int      kTmemCols  = 2 * kAccStride;
    constexpr int      kFeatOut   = (EPI == kEpiSwiGLU) ? 128 : 256;  // output columns of a pair's tile
    constexpr int      kFeatCta   = kFeatOut / 2;                     // of one CTA

    if (threadIdx.x == 0) {
        *fail_slot = 0;
        *epi_fail  = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);   // the leader's producer arrives once and expects the bytes of both CTAs
            mbar_init(&empty_bar[s], 1);  // one commit
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tfull_bar[s], 1);
            mbar_init(&tempty_bar[s], 256);  // the epilogue threads of both CTAs
        }
        fence_mbar_init();
        tma_prefetch_desc(&tmW);
        tma_prefetch_desc(&tmX);
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
            SwapWalker walk(args, kFeatOut, cluster, n_clusters);
            SwapTile   tc;
            int        stage = 0;
            uint32_t   phase = 0;
            bool       ok    = true;
            while (ok && walk.next(tc)) {
                // this CTA's weight rows: 128 output features, or 64 gate rows and the 64 up rows of the same features
                const int wrow = tc.group * args.rowsB + tc.nt * kFeatOut + static_cast<int>(crank) * kFeatCta;
                // this CTA's half of the tile's tokens
                const int xrow = tc.tok0 + static_cast<int>(crank) * (tc.ntok / 2);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, st, 1, stage, lim)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sw = smem + stage * S::kStageBytes;
                    uint8_t* sx = sw + S::kWBytes;
                    if (crank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * S::kStageBytes);
                    const uint32_t leader_full = mapa_u32(&full_bar[stage], 0);
                    if (EPI == kEpiSwiGLU) {  // the weight map's box is 64 rows
                        tma_load_2d_pair(sw, &tmW, leader_full, kb * kBK, wrow);
                        tma_load_2d_pair(sw + S::kWBytes / 2, &tmW, leader_full, kb * kBK, wrow + args.N);
                    }
                    else {
                        tma_load_2d_pair(sw, &tmW, leader_full, kb * kBK, wrow);
                    }
                    tma_load_2d_pair(sx, &tmX, leader_full, kb * kBK, xrow);
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
            SwapWalker walk(args, kFeatOut, cluster, n_clusters);
            SwapTile   tc;
            int        stage = 0;
            uint32_t   phase = 0;
            int        acc = 0;
            uint32_t   acc_phase = 0;
            bool       ok = true;
            while (ok && walk.next(tc)) {
                if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, st, 2, acc, lim)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t idesc  = make_idesc(kFmtBF16, kFmtBF16, kPairBM, static_cast<uint32_t>(tc.ntok));
                const uint32_t tmem_d = tmem_base + acc * kAccStride;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, st, 3, stage, lim)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t sw = smem_u32(smem + stage * S::kStageBytes);
                    const uint64_t da = make_kmajor_sw128_desc(sw);                // weights: the M operand
                    const uint64_t db = make_kmajor_sw128_desc(sw + S::kWBytes);   // tokens: the N operand
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
        // ------------------------------ epilogue (both CTAs, own TMEM lanes = own features) ------------------------------
        const int      quad = warp & 3;
        SwapWalker     walk(args, kFeatOut, cluster, n_clusters);
        SwapTile       tc;
        int            acc = 0;
        uint32_t       acc_phase = 0;
        unsigned int   block_no = 0;  // staged blocks so far: picks the staging buffer
        const uint32_t leader_tempty[2] = {mapa_u32(&tempty_bar[0], 0), mapa_u32(&tempty_bar[1], 0)};
        float*         stage_f = reinterpret_cast<float*>(epi_smem);
        while (walk.next(tc)) {
            if (!mbar_wait_relaxed(&tfull_bar[acc], acc_phase, st, 4, acc, lim)) {
                *fail_slot = 1;
                *epi_fail  = 1;
            }
            // The 128 epilogue threads meet at named barriers below, which have no time limit: they must leave the loop
            // together or not at all. A thread whose wait ran out says so before this barrier and everyone reads the
            // word after it (the word is written nowhere else, and the next write to it lies behind a later barrier).
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*epi_fail != 0) break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kAccStride;
            const int      feat0 = tc.nt * kFeatOut + static_cast<int>(crank) * kFeatCta;  // first output column of this CTA
#pragma unroll 1
            for (int c = 0; c < tc.ntok; c += 32) {
                float* blk = stage_f + (block_no & 1u) * (S::kBlockBytes / 4);
                ++block_no;
                uint32_t v[32];
                tmem_ld_32x32b_x32(taddr + c, v);
                tmem_ld_wait();
                // lane = feature (quad * 32 + lane of this CTA's 128 weight rows), v[i] = token c + i
#pragma unroll
                for (int i = 0; i < 32; ++i) blk[i * 128 + quad * 32 + lane] = __uint_as_float(v[i]);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                // token rows leave: warp w of the four takes tokens 8w .. 8w+7 of the block
                const int w = warp - 2;
                if (EPI == kEpiSwiGLU) {
                    // 64 output features per token and CTA: lanes 0..15 take one token, lanes 16..31 the next
                    const int piece = lane & 15;  // 4 features
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int tl  = w * 8 + j * 2 + (lane >> 4);
                        const int row = tc.tok0 + c + tl;
                        const float4 g = *reinterpret_cast<const float4*>(blk + tl * 128 + piece * 4);
                        const float4 u = *reinterpret_cast<const float4*>(blk + tl * 128 + 64 + piece * 4);
                        const int    col = feat0 + piece * 4;
                        if (row < tc.tok_end && col < args.N) {
                            uint2 o;
                            o.x = pack_bf16(silu(g.x) * u.x, silu(g.y) * u.y);
                            o.y = pack_bf16(silu(g.z) * u.z, silu(g.w) * u.w);
                            *reinterpret_cast<uint2*>(args.C + static_cast<long long>(row) * args.ldc + col) = o;
                        }
                    }
                }
                else {
                    // 128 output features per token and CTA: one token per warp instruction, 4 features per lane
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int tl  = w * 8 + j;
                        const int row = tc.tok0 + c + tl;
                        const int col = feat0 + lane * 4;
                        const float4 x = *reinterpret_cast<const float4*>(blk + tl * 128 + lane * 4);
                        if (row < tc.tok_end && col < args.N) {
                            float              scale = 1.0f;
                            unsigned long long dst;
                            bool               do_store = true;
                            if (EPI == kEpiScatterRows) {
                                const unsigned long long info   = args.row_info[row];
                                const unsigned int       region = static_cast<unsigned int>(info >> 48);
                                const unsigned long long slot   = info & 0xffffffffffffull;
                                const unsigned long long base   = region < 8 ? args.scatter_base[region] : 0ull;
                                do_store                        = base != 0ull && slot < args.scatter_slots;
                                dst = base + slot * args.scatter_row_bytes + static_cast<unsigned long long>(col) * 2;
                                if (do_store && args.row_scale) scale = args.row_scale[row];
                            }
                            else {
                                dst = reinterpret_cast<unsigned long long>(args.C + static_cast<long long>(row) * args.ldc + col);
                            }
                            if (do_store) {
                                uint2 o;
                                o.x = pack_bf16(x.x * scale, x.y * scale);
                                o.y = pack_bf16(x.z * scale, x.w * scale);
                                *reinterpret_cast<uint2*>(dst) = o;
                            }
                        }
                    }
                }
                // no second barrier: the next block goes to the other buffer, and a thread writes into this buffer again
                // only after the next block's barrier, which every thread passes after it has finished reading here
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
