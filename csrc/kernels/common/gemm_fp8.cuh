// Block-scaled fp8 (e4m3) GEMM on the tcgen05 tensor cores, bf16 output:
//
//   C[m, n] = sum over 128-wide K blocks kb of  sa[m, kb] * sb[n / 128, kb] * (Aq[m, kb] . Bq[n, kb])
//
// Aq [M, K] and Bq [N, K] are e4m3 bytes (K contiguous), sa [M, K/128] are the per-token 1x128 scales and
// sb [N/128, K/128] the 128x128 weight-block scales, both fp32: the DeepSeek-V3 recipe.
//
// The scale changes every K block, so the product cannot be left to accumulate in TMEM for the whole K
// loop. Two-level accumulation: a K block (128 bytes = one swizzle row = one pipeline stage) is FOUR
// tcgen05.mma.kind::f8f6f4 (K = 32 each) into a fresh TMEM partial; eight "promotion" warps read the
// partial (tcgen05.ld), multiply by sa * sb and add into fp32 registers, while the tensor core already
// fills the other partial (two partials of 128 x 256 fp32 = all 512 TMEM columns). One thread owns one row and
// 128 of the 256 columns (four 32-column reads and 128 FMAs per K block, 128 accumulators); at the end of the tile
// it converts and stores its 256 contiguous output bytes.
//
// The promotion is the limit, and it is the volume read back from TMEM, not the latency of a read: the tensor
// pipe is 39 % busy (8192^3 in 0.62 ms = 1769 TFLOP/s). Measured alternatives, all slower: 64-column reads (spill at
// the 168-register cap of ten warps: 1.20 ms), two overlapped 32-column reads (0.65 ms), 128 x 192 tiles with twelve
// warps of 64 columns each, no spills (0.69 ms). Doing the scaling in the tensor core (kind::mxf8f6f4 with UE8M0
// scale factors in TMEM) is what removes this read; it needs power-of-two scales.
//
// Roles per CTA (320 threads): warp 0 TMA producer, warp 1 TMEM owner + MMA issuer, warps 2..9
// promotion + epilogue (warp w reads TMEM lane quadrant w % 4, column slice (w - 2) / 4). Every wait is
// bounded and reports through the status page, as in the bf16 kernels. The all-gather roles of
// gemm_tc.cuh carry over: shard-major tiles, own shard read in place, tiles gated on arrival counters, one
// push warp that sends fp8 payload AND scales (half the NVLink bytes of the bf16 form).
#pragma once

#include "gemm_tc.cuh"

namespace slime {
namespace gemm {

constexpr int kF8BK       = 128;  // fp8 elements (= bytes) per K block
constexpr int kF8BN         = 256;  // tile width: two 128-column slices per TMEM lane quadrant
constexpr int kF8Cols       = 128;  // columns per promotion thread
constexpr int kF8PartStride = 256;  // TMEM columns between the two partials
constexpr int kF8Stages     = 4;
constexpr int kF8PromoWarps = 4 * (kF8BN / kF8Cols);
constexpr int kF8Threads    = (2 + kF8PromoWarps) * 32;
constexpr int kF8PromoThreads = kF8PromoWarps * 32;

struct F8Args {
    int M, N, K;
    __nv_bfloat16* C;
    long long      ldc;
    const float*   sa;        // [M, K/128] scales of A (for the all-gather form: of the GATHERED matrix)
    const float*   sa_local;  // all-gather form: scales of this rank's shard [ag_rows, K/128]
    const float*   sb;        // [ceil(N/128), K/128]
    Args           ag;        // all-gather roles (a_ready*, ag_*, status, wait_ns); the GEMM fields of it are unused
    // push of the scales next to the payload
    const uint8_t*     ag_src_scales;    // == sa_local
    unsigned long long ag_dst_scales[8]; // gathered scale matrix on every rank
};

template<bool AG>
struct SmemF8 {
    static constexpr int kABytes     = kBM * kF8BK;
    static constexpr int kBBytes     = kF8BN * kF8BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarBytes   = (2 * kF8Stages + 4 + kAgMaxBufs) * 8 + 16;
    static constexpr int kBase       = kF8Stages * kStageBytes + kBarBytes + 1024;
    static constexpr int kAgBufs = !AG ? 0 : ((kSmemLimit - kBase - 128) / kAgChunkBytes > kAgMaxBufs ? kAgMaxBufs : (kSmemLimit - kBase - 128) / kAgChunkBytes);
    static constexpr int kTotal  = kBase + (AG ? kAgBufs * kAgChunkBytes + 128 : 0);
};

// Push of one rank's fp8 shard and its scales, destination by destination, through the bulk-copy engine
// (same scheme as ag_push_bulk; a unit is 8 rows of payload followed by the 8 rows of scales).
__device__ __forceinline__ bool ag_push_bulk_f8(const F8Args& f, uint8_t* bufs, uint64_t* bars, int nb, int cta, int n_cta,
                                                KernelStatus* st, unsigned long long lim)
{
    const Args&              a           = f.ag;
    const unsigned long long row_bytes   = static_cast<unsigned long long>(f.K);
    const unsigned long long srow_bytes  = static_cast<unsigned long long>(f.K / kF8BK) * 4;
    const unsigned long long slice_bytes = row_bytes * kAgSliceRows;
    const unsigned long long sslice      = srow_bytes * kAgSliceRows;  // scales of one slice (a multiple of 16: 8 rows x 4 bytes x blocks)
    const int                slices      = a.ag_rows / kAgSliceRows;
    const int                units       = slices * a.ag_world;
    const int                pchunks     = static_cast<int>((slice_bytes + kAgChunkBytes - 1) / kAgChunkBytes);
    const int                schunks     = static_cast<int>((sslice + kAgChunkBytes - 1) / kAgChunkBytes);
    const int                chunks      = pchunks + schunks;
    const uint8_t*           src_base    = reinterpret_cast<const uint8_t*>(a.ag_src);
    // chunk c of slice sl: source address, destination offset inside the rank's slice, bytes
    auto chunk_src = [&](int sl, int c, uint32_t& bytes) -> const uint8_t* {
        if (c < pchunks) {
            const unsigned long long off  = static_cast<unsigned long long>(c) * kAgChunkBytes;
            const unsigned long long left = slice_bytes - off;
            bytes = left < kAgChunkBytes ? static_cast<uint32_t>(left) : kAgChunkBytes;
            return src_base + static_cast<unsigned long long>(sl) * slice_bytes + off;
        }
        const unsigned long long off  = static_cast<unsigned long long>(c - pchunks) * kAgChunkBytes;
        const unsigned long long left = sslice - off;
        bytes = left < kAgChunkBytes ? static_cast<uint32_t>(left) : kAgChunkBytes;
        return f.ag_src_scales + static_cast<unsigned long long>(sl) * sslice + off;
    };
    auto signal_unit = [&](int u) {
        const int p  = (a.ag_rank + 1 + u / slices) % a.ag_world;
        const int sl = u % slices;
        fence_proxy_async();
        fence_acq_rel_sys();
        unsigned long long* fl = reinterpret_cast<unsigned long long*>(a.ag_flags[p]) + a.ag_rank * (a.ag_rows / kBM)
                                 + sl / (kBM / kAgSliceRows);
        red_add_release_sys(fl, 1ull);
    };
    int lu = cta, lc = 0, n_ld = 0;
    auto issue_load = [&]() {
        const int      b = n_ld % nb;
        uint32_t       bytes;
        const uint8_t* src = chunk_src(lu % slices, lc, bytes);
        mbar_arrive_expect_tx(&bars[b], bytes);
        bulk_load_g2s(bufs + b * kAgChunkBytes, src, bytes, &bars[b]);
        ++n_ld;
        if (++lc == chunks) {
            lc = 0;
            lu += n_cta;
        }
    };
    while (n_ld < nb && lu < units) issue_load();
    int n_st = 0, pending = -1;
    for (int u = cta; u < units; u += n_cta) {
        const int p  = (a.ag_rank + 1 + u / slices) % a.ag_world;
        const int sl = u % slices;
        uint8_t*  dst  = reinterpret_cast<uint8_t*>(a.ag_dst[p]) + (static_cast<unsigned long long>(a.ag_rank) * slices + sl) * slice_bytes;
        uint8_t*  sdst = reinterpret_cast<uint8_t*>(f.ag_dst_scales[p]) + (static_cast<unsigned long long>(a.ag_rank) * slices + sl) * sslice;
        for (int c = 0; c < chunks; ++c) {
            const int b = n_st % nb;
            if (!mbar_wait_relaxed(&bars[b], (n_st / nb) & 1, st, 12, b, lim)) return false;
            uint32_t bytes;
            chunk_src(sl, c, bytes);
            uint8_t* d = c < pchunks ? dst + static_cast<unsigned long long>(c) * kAgChunkBytes
                                     : sdst + static_cast<unsigned long long>(c - pchunks) * kAgChunkBytes;
            bulk_store_s2g(d, bufs + b * kAgChunkBytes, bytes);
            tma_store_commit();
            ++n_st;
            if (n_st >= 2 && lu < units) {
                tma_store_wait_read<1>();
                issue_load();
            }
            if (pending >= 0 && c == 1) {
                tma_store_wait<2>();
                signal_unit(pending);
                pending = -1;
            }
        }
        if (chunks < 3) {
            tma_store_wait<0>();
            signal_unit(u);
        }
        else {
            pending = u;
        }
    }
    tma_store_wait<0>();
    if (pending >= 0) signal_unit(pending);
    return true;
}

// Tile sequence of one CTA: m fastest, or shard-major in the all-gather form (128-row tiles).
struct F8Walker {
    const F8Args& f;
    int           mtiles, ntiles, total, t;
    __device__ F8Walker(const F8Args& args): f(args)
    {
        mtiles = (f.M + kBM - 1) / kBM;
        ntiles = (f.N + kF8BN - 1) / kF8BN;
        total  = mtiles * ntiles;
        t      = blockIdx.x;
    }
    __device__ bool next(int& row0, int& nt)
    {
        if (t >= total) return false;
        int mt;
        if (f.ag.ag_shard_order) {
            const int per       = f.ag.ag_rows / kBM;
            const int per_shard = per * ntiles;
            const int j         = t / per_shard;
            const int rem       = t - j * per_shard;
            const int shard     = ((f.ag.ag_rank - j) % f.ag.ag_world + f.ag.ag_world) % f.ag.ag_world;
            nt                  = rem / per;
            mt                  = shard * per + rem % per;
        }
        else {
            mt = t % mtiles;
            nt = t / mtiles;
        }
        row0 = mt * kBM;
        t += gridDim.x;
        return true;
    }
};

template<bool AG>
__global__ void __launch_bounds__(kF8Threads + (AG ? kAgThreads : 0), 1)
gemm_fp8_blockscaled_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                            const __grid_constant__ CUtensorMap tmAL, const F8Args f)
{
    using S = SmemF8<AG>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    uint64_t* full_bar   = reinterpret_cast<uint64_t*>(smem + kF8Stages * S::kStageBytes);
    uint64_t* empty_bar  = full_bar + kF8Stages;
    uint64_t* pfull_bar  = empty_bar + kF8Stages;  // [2] partial product ready
    uint64_t* pempty_bar = pfull_bar + 2;          // [2] partial product consumed
    uint64_t* ag_bar     = pempty_bar + 2;
    uint32_t* tmem_slot  = reinterpret_cast<uint32_t*>(ag_bar + kAgMaxBufs);
    volatile uint32_t* fail_slot = tmem_slot + 1;
    uint8_t*  ag_bufs    = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem + kF8Stages * S::kStageBytes + S::kBarBytes) + 127) & ~uintptr_t(127));

    const int          warp    = threadIdx.x >> 5;
    const int          lane    = threadIdx.x & 31;
    const int          kblocks = (f.K + kF8BK - 1) / kF8BK;
    KernelStatus*      st      = f.ag.status;
    const unsigned long long lim = f.ag.wait_ns ? f.ag.wait_ns : kDefaultWaitNs;
    constexpr int      kTmemCols = 512;

    if (threadIdx.x == 0) {
        *fail_slot = 0;
        for (int s = 0; s < kF8Stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&pfull_bar[s], 1);
            mbar_init(&pempty_bar[s], kF8PromoThreads);
        }
        if (AG)
            for (int s = 0; s < kAgMaxBufs; ++s) mbar_init(&ag_bar[s], 1);
        fence_mbar_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if (AG) tma_prefetch_desc(&tmAL);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            F8Walker walk(f);
            int      row0, nt, stage = 0;
            uint32_t phase = 0;
            bool     ok    = true;
            while (ok && walk.next(row0, nt)) {
                const CUtensorMap* mapA = &tmA;
                int                arow = row0;
                bool               gate = f.ag.a_ready != nullptr;
                if (AG && f.ag.ag_local_direct && row0 / f.ag.ag_rows == f.ag.ag_rank) {
                    mapA = &tmAL;
                    arow = row0 - f.ag.ag_rank * f.ag.ag_rows;
                    gate = false;
                }
                if (gate) {
                    const int fl = row0 / f.ag.a_ready_rows;
                    ok = wait_flag_ge(f.ag.a_ready + fl, f.ag.a_ready_target, st, 10, fl, lim);
                    if (!ok) break;
                    fence_proxy_async();
                }
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, st, 1, stage, lim)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * S::kStageBytes;
                    uint8_t* sb = sa + S::kABytes;
                    mbar_arrive_expect_tx(&full_bar[stage], S::kStageBytes);
                    tma_load_2d(sa, mapA, &full_bar[stage], kb * kF8BK, arow);
                    tma_load_2d(sb, &tmB, &full_bar[stage], kb * kF8BK, nt * kF8BN);
                    tma_load_2d(sb + S::kBBytes / 2, &tmB, &full_bar[stage], kb * kF8BK, nt * kF8BN + kF8BN / 2);
                    if (++stage == kF8Stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) *fail_slot = 1;
        }
    }
    else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            F8Walker walk(f);
            int      row0, nt, stage = 0;
            uint32_t phase = 0;
            int      part = 0;
            uint32_t part_phase = 0;
            bool     ok = true;
            constexpr uint32_t idesc = make_idesc(kFmtE4M3, kFmtE4M3, kBM, kF8BN);
            while (ok && walk.next(row0, nt)) {
                for (int kb = 0; kb < kblocks && ok; ++kb) {
                    if (!mbar_wait(&pempty_bar[part], part_phase ^ 1, st, 2, part, lim) || !mbar_wait(&full_bar[stage], phase, st, 3, stage, lim)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t tmem_d = tmem_base + part * kF8PartStride;
                    const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
                    const uint32_t sb = sa + S::kABytes;
                    const uint64_t da = make_kmajor_sw128_desc(sa);
                    const uint64_t db = make_kmajor_sw128_desc(sb);
#pragma unroll
                    for (int k = 0; k < kF8BK / 32; ++k) umma_f8f6f4(tmem_d, da + 2 * k, db + 2 * k, idesc, k != 0);
                    umma_commit(&empty_bar[stage]);
                    umma_commit(&pfull_bar[part]);
                    if (++stage == kF8Stages) {
                        stage = 0;
                        phase ^= 1;
                    }
                    if (++part == 2) {
                        part = 0;
                        part_phase ^= 1;
                    }
                }
            }
            if (!ok) *fail_slot = 1;
        }
    }
    else if (AG && warp >= 2 + kF8PromoWarps) {
        if (f.ag.ag_src != nullptr && lane == 0) {
            if (!ag_push_bulk_f8(f, ag_bufs, ag_bar, S::kAgBufs, blockIdx.x, gridDim.x, st, lim)) *fail_slot = 1;
        }
    }
    else {
        // ------------------------------ promotion + epilogue ------------------------------
        const int quad = warp & 3;
        const int grp  = (warp - 2) >> 2;  // which 64-column slice of the tile
        const int srow = kblocks;          // scales per row
        F8Walker  walk(f);
        int       row0, nt;
        int       part = 0;
        uint32_t  part_phase = 0;
        bool      ok = true;
        while (ok && walk.next(row0, nt)) {
            const int  row   = row0 + quad * 32 + lane;
            const bool valid = row < f.M;
            const int  crow  = valid ? row : f.M - 1;
            const float* sa_row;
            if (AG && f.ag.ag_local_direct && row0 / f.ag.ag_rows == f.ag.ag_rank) {
                sa_row = f.sa_local + static_cast<long long>(crow - f.ag.ag_rank * f.ag.ag_rows) * srow;
            }
            else {
                sa_row = f.sa + static_cast<long long>(crow) * srow;
                if (f.ag.a_ready) {
                    // the scales of a gathered shard arrive with its payload: this thread reads them with plain loads,
                    // so it has to see the arrival counter itself (the producer's wait orders only the TMA loads)
                    const int fl = row0 / f.ag.a_ready_rows;
                    if (!wait_flag_ge(f.ag.a_ready + fl, f.ag.a_ready_target, st, 11, fl, lim)) {
                        ok = false;
                        break;
                    }
                }
            }
            const int    nblk   = (nt * kF8BN + grp * kF8Cols) / 128;  // a 64-column slice never straddles a 128-wide scale block
            const int    nblk_c = nblk < (f.N + 127) / 128 ? nblk : (f.N + 127) / 128 - 1;
            const float* sb_row = f.sb + static_cast<long long>(nblk_c) * srow;
            float acc[kF8Cols];
#pragma unroll
            for (int i = 0; i < kF8Cols; ++i) acc[i] = 0.0f;
            float s_next = sa_row[0] * sb_row[0];
            for (int kb = 0; kb < kblocks; ++kb) {
                const float s = s_next;
                if (kb + 1 < kblocks) s_next = sa_row[kb + 1] * sb_row[kb + 1];
                if (!mbar_wait(&pfull_bar[part], part_phase, st, 4, part, lim)) {
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + part * kF8PartStride + grp * kF8Cols;
#pragma unroll
                for (int c = 0; c < kF8Cols / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(s, __uint_as_float(v[i]), acc[c * 32 + i]);
                }
                tc_fence_before_sync();
                mbar_arrive(&pempty_bar[part]);
                if (++part == 2) {
                    part = 0;
                    part_phase ^= 1;
                }
            }
            if (!ok) break;
            const int col0 = nt * kF8BN + grp * kF8Cols;
            if (valid) {
                __nv_bfloat16* crow_ptr = f.C + static_cast<long long>(row) * f.ldc + col0;
                const int      cols     = f.N - col0;  // a multiple of 8 (N % 32 == 0)
#pragma unroll
                for (int i = 0; i < kF8Cols / 8; ++i) {
                    if (i * 8 < cols) {
                        uint4 o = make_uint4(pack_bf16(acc[8 * i], acc[8 * i + 1]), pack_bf16(acc[8 * i + 2], acc[8 * i + 3]),
                                             pack_bf16(acc[8 * i + 4], acc[8 * i + 5]), pack_bf16(acc[8 * i + 6], acc[8 * i + 7]));
                        *reinterpret_cast<uint4*>(crow_ptr + 8 * i) = o;
                    }
                }
            }
        }
        if (!ok) *fail_slot = 1;
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        if (*fail_slot != 0) {
            const unsigned long long t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace gemm
}  // namespace slime
