// Persistent, warp-specialised bf16 GEMM main loop on the 5th-generation tensor
// cores: TMA (128-byte swizzle) -> shared memory ring -> tcgen05.mma (one issuing
// thread) -> fp32 accumulators in TMEM (double buffered) -> tcgen05.ld epilogue.
//
//   C[g] (rows of group g, N) = A[g] (rows of group g, K) * B[g] (N, K)^T
//
// A is one row-major [M_total, K] matrix whose rows are partitioned into groups
// by a device-side prefix array; B is row-major [groups * rowsB, K] ("K-major",
// the nn.Linear layout). Tiles are 128 x BN x 64. A tile that crosses the end of
// its group computes garbage rows that the epilogue never stores, so groups need
// no row padding.
//
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner and MMA
// issuer, warps 2..5 = epilogue (each owns the 32 TMEM lanes of its quadrant).
// Every wait is bounded; a timeout is recorded in the status page and the CTA
// drains, frees its TMEM and returns.
#pragma once

#include "fp8.cuh"
#include "ptx.cuh"

namespace slime {
namespace gemm {

constexpr int kBM      = 128;
constexpr int kBK      = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int kThreads = 192;
constexpr int kEpiRowPitch = 128;  // one 128-byte slot per tile row; the 16-byte pieces of a slot are XOR-swizzled with the row

enum Epilogue : int {
    kEpiStore  = 0,  // C = acc (bf16)
    kEpiSwiGLU = 1,  // tile columns [0,BN/2) are gate, [BN/2,BN) are up: C = silu(gate) * up
    kEpiScatterRows = 2,  // row r goes to scatter_base[info >> 48] + (info & 2^48-1) * scatter_row_bytes (peer memory allowed)
};

struct Args {
    int M_total;  // rows in A (upper bound for every group end)
    int N;        // output columns per group (for SwiGLU: the intermediate size)
    int K;
    int rowsB;  // rows of B per group (N, or 2N for SwiGLU where gate rows precede up rows)
    int num_groups;
    const int* group_offsets;  // [num_groups + 1] device prefix of rows, or nullptr for one group [0, M_total)
    __nv_bfloat16* C;
    long long      ldc;
    // kEpiScatterRows: per-row destination (region index << 48 | row slot inside that region) and optional weight
    const unsigned long long* row_info;   // [M_total]; a region index >= 8 or a slot >= scatter_slots drops the row
    const float*              row_scale;  // [M_total] or nullptr
    unsigned long long        scatter_base[8];  // base address of each destination region (0 = absent)
    unsigned long long        scatter_row_bytes;
    unsigned long long        scatter_slots;
    // optional per-128-row A readiness flags (all-gather -> GEMM): tile rows [128*i, 128*i+128)
    // may be read once a_ready[i / a_ready_div] >= a_ready_target
    const unsigned long long* a_ready;
    int                       a_ready_rows;  // rows covered by one flag
    unsigned long long        a_ready_target;
    int                       m_tile_rotate;  // start the m-tile order at this tile (own shard first)
    // all-gather -> GEMM (fused form): extra warps of every CTA copy slices of this rank's shard of A
    // into every rank's gathered matrix and bump that rank's arrival counters
    const uint4*              ag_src;          // this rank's shard [ag_rows, K] (nullptr = no push in this kernel)
    int                       ag_rows;         // rows per shard (multiple of 128)
    int                       ag_rank, ag_world;
    int                       ag_shard_order;  // visit m tiles shard by shard: own, rank-1, rank-2, ...
    int                       ag_local_direct; // tiles of the own shard read ag_src through the third tensor map and wait for nothing
    unsigned long long        ag_dst[8];       // address of the gathered A on every rank
    unsigned long long        ag_flags[8];     // address of the arrival counters (u64 per 128 rows) on every rank
    // optional per-group readiness words (streamed expert-parallel receive): the rows of group g may be read once
    // group_ready[g] >= the step number, which is group_ready_target or, when group_ready_epoch is set, the value
    // found there when the kernel starts (a device-resident step counter, so that a captured step replays)
    const unsigned long long* group_ready;
    unsigned long long        group_ready_target;
    const unsigned long long* group_ready_epoch;
    // optional dynamic tile scheduler (u32 [2], zero before the first launch; the kernel leaves it zero): CTAs take
    // tiles from a shared counter instead of every gridDim-th tile, so a CTA that starts late or shares its SM with
    // other kernels simply takes fewer tiles
    unsigned int*             tile_counter;
    // optional trace (u64 [2 * num_groups + gridDim.x], device memory): CTA 0's producer records, per group, when it
    // began to wait for the group and when the group was ready (globaltimer ns); behind that, every CTA's start time
    unsigned long long*       group_trace;
    // weight-streaming launches (few rows per group): the producer asks L2 for the B boxes this many K blocks ahead of
    // its loads, into the CTA's next tile too, so that more bytes are in flight from HBM than the shared-memory ring
    // holds (0 = off; static tile order only). Measured on the weight-streaming shapes it LOSES at every distance (256
    // experts x ~128 rows: 5.31 TB/s of weights without, 4.68 / 4.03 / 3.43 / 3.11 TB/s at 4 / 8 / 16 / 32 blocks; 32 x 32
    // rows: 5.52 against 5.02 and less): 148 CTAs with four 48 KB stages already keep HBM busy, and the extra requests
    // only disturb the order in which it is read. Off everywhere; kept as an option of the launcher.
    int                       w_prefetch;
    // A operand as e4m3 with 1x128 scales (kernels instantiated with A8): the tile is expanded to bf16 in shared memory
    const float*              a_scale;         // [M_total, K / 128]
    KernelStatus*             status;
    unsigned long long        wait_ns;
};

constexpr int kTileRing     = 4;     // tile indices in flight between the producer and the roles that follow it
constexpr int kAgChunkBytes = 4096;  // staging buffer of the in-kernel all-gather push
constexpr int kAgMaxBufs    = 6;
constexpr int kSmemLimit    = 227 * 1024;

// AROWS: rows of A that a stage holds (128, or 64 for launches whose groups are small: the MMA still reads 128 rows, the
// upper 64 from whatever follows in the stage, and their results are never stored)
template<int BN, int STAGES, bool AG = false, bool A8 = false, int AROWS = kBM>
struct Smem {
    static constexpr int kABytes     = AROWS * kBK * 2;
    static constexpr int kBBytes     = BN * kBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kRawBytes   = A8 ? kBM * kBK : 0;  // e4m3 A tile of a stage as it arrives, before expansion
    static constexpr int kBarBytes   = (3 * STAGES + 4 + kAgMaxBufs + 2 * kTileRing) * 8 + 16 + kTileRing * 4;
    static constexpr int kEpiBytes   = 128 * kEpiRowPitch;  // one 128-byte slot per tile row
    static constexpr int kBase       = STAGES * (kStageBytes + kRawBytes) + kEpiBytes + kBarBytes + 1024;  // + alignment slack
    // the push stages its chunks in whatever shared memory the tile ring leaves free
    static constexpr int kAgBufs = !AG ? 0 : ((kSmemLimit - kBase - 128) / kAgChunkBytes > kAgMaxBufs ? kAgMaxBufs : (kSmemLimit - kBase - 128) / kAgChunkBytes);
    static constexpr int kTotal  = kBase + (AG ? kAgBufs * kAgChunkBytes + 128 : 0);
    static_assert(!AG || kAgBufs >= 2, "no room for the push buffers");
};

struct TileCoord {
    int group;
    int row0;     // first row of the tile in A / C
    int row_end;  // one past the last valid row of the group
    int nt;       // n-tile index inside the group
};

// Walks the persistent tile sequence blockIdx.x, blockIdx.x + gridDim.x, ...
// Order inside a group: m fastest, so CTAs running at the same time share B tiles in L2.
struct TileWalker {
    const Args& a;
    int         ntiles_n;
    int         t;          // next linear tile for this CTA
    int         g;          // current group
    int         cum;        // tiles before group g
    int         g_begin, g_end, g_mtiles;
    int         tile_rows;  // rows of a tile: 128, or 64 in the short-A instantiations

    __device__ TileWalker(const Args& args, int bn_out, int rows_per_tile = kBM): a(args), tile_rows(rows_per_tile)
    {
        ntiles_n = (a.N + bn_out - 1) / bn_out;
        t        = blockIdx.x;
        g        = -1;
        cum      = 0;
        g_begin = g_end = g_mtiles = 0;
        advance_group();
    }
    __device__ void advance_group()
    {
        ++g;
        if (g < a.num_groups) {
            g_begin  = a.group_offsets ? a.group_offsets[g] : 0;
            g_end    = a.group_offsets ? a.group_offsets[g + 1] : a.M_total;
            if (g_end > a.M_total) g_end = a.M_total;
            if (g_begin > g_end) g_begin = g_end;
            g_mtiles = (g_end - g_begin + tile_rows - 1) / tile_rows;
        }
    }
    __device__ bool next(TileCoord& c)
    {
        const bool have = at(t, c);
        t += gridDim.x;
        return have;
    }
    // Coordinates of linear tile `lt`; calls must come with non-decreasing lt. False past the last tile.
    __device__ bool at(int lt, TileCoord& c)
    {
        const int t = lt;
        while (g < a.num_groups) {
            const int tiles_g = g_mtiles * ntiles_n;
            if (t < cum + tiles_g) {
                const int local = t - cum;
                int       mt, nt;
                if (a.ag_shard_order) {
                    // shard-major order: every tile of the local shard first, then the shard of rank-1, rank-2, ...
                    // (the order in which the shards finish arriving), n tiles before m tiles inside a shard
                    const int per       = a.ag_rows / kBM;
                    const int per_shard = per * ntiles_n;
                    const int j         = local / per_shard;
                    const int rem       = local - j * per_shard;
                    const int shard     = ((a.ag_rank - j) % a.ag_world + a.ag_world) % a.ag_world;
                    nt                  = rem / per;
                    mt                  = shard * per + rem % per;
                }
                else {
                    mt = local % g_mtiles;
                    if (a.m_tile_rotate) mt = (mt + a.m_tile_rotate) % g_mtiles;
                    nt = local / g_mtiles;
                }
                c.group   = g;
                c.row0    = g_begin + mt * tile_rows;
                c.row_end = g_end;
                c.nt      = nt;
                return true;
            }
            cum += tiles_g;
            advance_group();
        }
        return false;
    }
};

// Where a role gets its next tile index from: every gridDim-th tile (static), or the shared-memory ring that the
// producer fills from the global tile counter (dynamic). One instance per thread that walks tiles.
struct TileFeed {
    bool      dynamic;
    int       t_static;
    int*      ring;
    uint64_t* full;
    uint64_t* empty;
    int       slot  = 0;
    uint32_t  phase = 0;
    __device__ TileFeed(const Args& a, int* r, uint64_t* f, uint64_t* e):
        dynamic(a.tile_counter != nullptr), t_static(blockIdx.x), ring(r), full(f), empty(e)
    {
    }
    __device__ void advance()
    {
        if (++slot == kTileRing) {
            slot = 0;
            phase ^= 1;
        }
    }
    // Consumer side: the next tile index, -1 at the end (or when the wait ran out, with ok = false).
    __device__ int take(KernelStatus* st, unsigned long long lim, bool& ok)
    {
        if (!dynamic) {
            const int t = t_static;
            t_static += gridDim.x;
            return t;
        }
        if (!mbar_wait(&full[slot], phase, st, 6, slot, lim)) {
            ok = false;
            return -1;
        }
        const int t = ring[slot];
        mbar_arrive(&empty[slot]);
        advance();
        return t;
    }
    // Producer side: claims the next tile index and, in dynamic mode, hands it (or the end mark) to the ring.
    __device__ int claim(const Args& a)
    {
        if (!dynamic) {
            const int t = t_static;
            t_static += gridDim.x;
            return t;
        }
        return static_cast<int>(atomicAdd(a.tile_counter, 1u));
    }
    __device__ bool publish(int t, KernelStatus* st, unsigned long long lim)
    {
        if (!dynamic) return true;
        if (!mbar_wait(&empty[slot], phase ^ 1, st, 7, slot, lim)) return false;
        ring[slot] = t;
        mbar_arrive(&full[slot]);
        advance();
        return true;
    }
};

__device__ __forceinline__ float silu(float x)
{
    return x / (1.0f + __expf(-x));
}

// One 64-column piece of 32 result rows leaves the SM: every lane has its row's 128 bytes (packed bf16) in registers,
// writes them to its slot, and the warp then stores row by row, eight lanes per row and 16 bytes per lane, so that
// every store instruction writes four whole 128-byte lines (local or peer memory). Piece p of row r sits at
// p ^ (r & 7) inside the slot, which keeps both the row-wise writes and the line-wise reads free of bank conflicts
// without padding. `dst` is this lane's row address for the piece, `do_store` whether its row is written at all,
// `cols` how many of the 64 columns exist (a multiple of 8). Must be called by all 32 lanes.
// (One bulk copy per row and piece, which this replaces, costs about 32 cycles of the SM's copy engine each: 1024 of
// them per 128 x 512 tile took as long as a quarter of the main loop.)
__device__ __forceinline__ void epi_store_piece(uint8_t* my_slot, const uint8_t* warp_slots, const uint32_t (&o)[32],
                                                unsigned long long dst, bool do_store, int cols, int lane)
{
    uint4* sp = reinterpret_cast<uint4*>(my_slot);
#pragma unroll
    for (int i = 0; i < 8; ++i) sp[i ^ (lane & 7)] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
    __syncwarp();
    const int sub = lane >> 3, piece = lane & 7;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int                r  = i * 4 + sub;
        const unsigned long long d  = __shfl_sync(0xffffffffu, dst, r);
        const int                ok = __shfl_sync(0xffffffffu, do_store ? 1 : 0, r);
        if (ok && piece * 8 < cols) {
            const uint4 v = *reinterpret_cast<const uint4*>(warp_slots + r * kEpiRowPitch + ((piece ^ (r & 7)) << 4));
            *reinterpret_cast<uint4*>(d + static_cast<unsigned long long>(piece) * 16) = v;
        }
    }
    __syncwarp();  // the slots may be overwritten by the next piece
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// All-gather push executed by `nthreads` threads (tid in [0, nthreads)) that share named barrier
// `bar_id`. A unit is (destination, 8-row slice of the local shard); units are numbered destination by
// destination (rank+1, rank+2, ..., and this rank itself last), so the CTAs of the grid, which take
// units round robin, all work on the same destination at the same time: every rank then receives from
// one source at a time at full link rate, and the shards complete in the order in which the tiles
// consume them. Every finished unit adds 1 to the destination's counter of the 128-row chunk it
// belongs to, so a chunk is complete at 16 * step.
constexpr int kAgSliceRows = 8;
__device__ __forceinline__ void ag_push_units(const Args& a, int tid, int nthreads, int bar_id, int cta, int n_cta)
{
    const unsigned long long row_vecs = static_cast<unsigned long long>(a.K) * 2 / 16;
    const unsigned long long slice_v  = row_vecs * kAgSliceRows;
    const int                slices   = a.ag_rows / kAgSliceRows;
    const int                units    = slices * a.ag_world;
    for (int u = cta; u < units; u += n_cta) {
        const int    p   = (a.ag_rank + 1 + u / slices) % a.ag_world;
        const int    sl  = u % slices;
        const uint4* src = a.ag_src + sl * slice_v;
        uint4* dst = reinterpret_cast<uint4*>(a.ag_dst[p]) + (static_cast<unsigned long long>(a.ag_rank) * slices + sl) * slice_v;
        unsigned long long i = tid;
        for (; i + 7ull * nthreads < slice_v; i += 8ull * nthreads) {
            uint4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = src[i + j * nthreads];
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[i + j * nthreads] = v[j];
        }
        for (; i < slice_v; i += nthreads) dst[i] = src[i];
        asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
        if (tid == 0) {
            fence_acq_rel_sys();
            unsigned long long* f = reinterpret_cast<unsigned long long*>(a.ag_flags[p])
                                    + a.ag_rank * (a.ag_rows / kBM) + sl / (kBM / kAgSliceRows);
            red_add_release_sys(f, 1ull);
        }
    }
}

// The same push through the bulk-copy engine, executed by ONE thread: chunks of the local shard are
// loaded into a ring of shared-memory buffers (completion on an mbarrier each) and handed on to the
// destination with shared -> global bulk copies, which also reach peer memory. Loads run ahead of
// stores by the ring depth; a buffer is reloaded once the copy engine has read it. A unit's counter is
// bumped when its copies are complete, which is checked two chunks into the next unit so that the
// pipeline never drains. Returns false when a wait ran out.
__device__ __forceinline__ bool ag_push_bulk(const Args& a, uint8_t* bufs, uint64_t* bars, int nb, int cta, int n_cta,
                                             KernelStatus* st, unsigned long long lim)
{
    const unsigned long long slice_bytes = static_cast<unsigned long long>(a.K) * 2 * kAgSliceRows;
    const int                slices      = a.ag_rows / kAgSliceRows;
    const int                units       = slices * a.ag_world;
    const int                chunks      = static_cast<int>((slice_bytes + kAgChunkBytes - 1) / kAgChunkBytes);
    const uint8_t*           src_base    = reinterpret_cast<const uint8_t*>(a.ag_src);
    auto chunk_bytes = [&](int c) -> uint32_t {
        const unsigned long long left = slice_bytes - static_cast<unsigned long long>(c) * kAgChunkBytes;
        return left < kAgChunkBytes ? static_cast<uint32_t>(left) : kAgChunkBytes;
    };
    auto signal_unit = [&](int u) {
        const int p  = (a.ag_rank + 1 + u / slices) % a.ag_world;
        const int sl = u % slices;
        fence_proxy_async();
        fence_acq_rel_sys();
        unsigned long long* f = reinterpret_cast<unsigned long long*>(a.ag_flags[p]) + a.ag_rank * (a.ag_rows / kBM)
                                + sl / (kBM / kAgSliceRows);
        red_add_release_sys(f, 1ull);
    };
    int lu = cta, lc = 0, n_ld = 0;  // load cursor
    auto issue_load = [&]() {
        const int      b     = n_ld % nb;
        const uint32_t bytes = chunk_bytes(lc);
        mbar_arrive_expect_tx(&bars[b], bytes);
        bulk_load_g2s(bufs + b * kAgChunkBytes, src_base + static_cast<unsigned long long>(lu % slices) * slice_bytes
                                                     + static_cast<unsigned long long>(lc) * kAgChunkBytes, bytes, &bars[b]);
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
        uint8_t*  dst = reinterpret_cast<uint8_t*>(a.ag_dst[p]) + (static_cast<unsigned long long>(a.ag_rank) * slices + sl) * slice_bytes;
        for (int c = 0; c < chunks; ++c) {
            const int b = n_st % nb;
            if (!mbar_wait_relaxed(&bars[b], (n_st / nb) & 1, st, 12, b, lim)) return false;
            bulk_store_s2g(dst + static_cast<unsigned long long>(c) * kAgChunkBytes, bufs + b * kAgChunkBytes, chunk_bytes(c));
            tma_store_commit();
            ++n_st;
            if (n_st >= 2 && lu < units) {
                tma_store_wait_read<1>();  // the buffer of the previous chunk has been read: load the next chunk into it
                issue_load();
            }
            if (pending >= 0 && c == 1) {
                tma_store_wait<2>();  // everything older than the last two copies has landed: that covers the previous unit
                signal_unit(pending);
                pending = -1;
            }
        }
        if (chunks < 3) {
            signal_unit(u);
        }
        else {
            pending = u;
        }
    }
    if (pending >= 0) signal_unit(pending);
    return true;
}

constexpr int kAgThreads = 32;

static __global__ void __launch_bounds__(256) ag_push_only_kernel(const Args args)
{
    ag_push_units(args, threadIdx.x, blockDim.x, 1, blockIdx.x, gridDim.x);
}

constexpr int kCvtThreads = 128;  // A8 kernels: four more warps expand the e4m3 A tile of every stage to bf16

// A8 = true: tmA describes A as e4m3 bytes [M_total, K] (box 128 rows x 64 bytes, no swizzle) and args.a_scale its 1x128
// scales. The producer lands the raw tile in a staging area; four converter warps (one thread per tile row) multiply
// by the row's scale, round to bf16 exactly as the stand-alone dequantisation kernel does, and write the tile in the
// 128-byte-swizzled K-major layout the MMA descriptor expects; the "full" barrier of the stage then needs the B bytes
// AND the converters' arrival. This removes the dequantisation pass over the received rows and halves the A traffic,
// but the raw tile costs a pipeline stage (3 instead of 4) and the expansion sits between the load and the MMA: in the
// weight-streaming regime (256 experts x 128 rows on one GPU) the kernel was measured 38 % slower than the 4-stage one,
// more than the separate pass costs, so callers keep the two-pass path by default.
template<int BN, int STAGES, int EPI, bool AG = false, bool A8 = false, int AROWS = kBM>
__global__ void __launch_bounds__(kThreads + (AG ? kAgThreads : 0) + (A8 ? kCvtThreads : 0), 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmAL, const Args args)
{
    static_assert(!(AG && A8), "the all-gather form takes bf16 activations");
    static_assert(AROWS == kBM || (AROWS == 64 && !AG && !A8), "short A tiles: 64 rows, grouped bf16 launches only");
    using S = Smem<BN, STAGES, AG, A8, AROWS>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    uint8_t*  raw_smem   = smem + STAGES * S::kStageBytes;             // [STAGES][kRawBytes] (A8 only)
    uint8_t*  epi_smem   = raw_smem + STAGES * S::kRawBytes;
    uint64_t* full_bar   = reinterpret_cast<uint64_t*>(epi_smem + S::kEpiBytes);
    uint64_t* empty_bar  = full_bar + STAGES;
    uint64_t* raw_bar    = empty_bar + STAGES;  // [STAGES] raw A tile landed (A8 only)
    uint64_t* tfull_bar  = raw_bar + STAGES;    // [2] accumulator ready
    uint64_t* tempty_bar = tfull_bar + 2;       // [2] accumulator drained
    uint64_t* ag_bar     = tempty_bar + 2;      // [kAgMaxBufs] push chunk loaded
    uint64_t* tr_full    = ag_bar + kAgMaxBufs; // [kTileRing] tile index published (dynamic scheduler)
    uint64_t* tr_empty   = tr_full + kTileRing; // [kTileRing] tile index taken by the MMA thread and every epilogue thread
    uint32_t* tmem_slot  = reinterpret_cast<uint32_t*>(tr_empty + kTileRing);
    int*      tile_ring  = reinterpret_cast<int*>(tmem_slot + 2);
    uint8_t*  ag_bufs    = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(epi_smem + S::kEpiBytes + S::kBarBytes) + 127) & ~uintptr_t(127));
    volatile uint32_t* fail_slot = tmem_slot + 1;  // set by any role whose wait ran out

    const int          warp    = threadIdx.x >> 5;
    const int          lane    = threadIdx.x & 31;
    const int          kblocks = (args.K + kBK - 1) / kBK;
    KernelStatus*      st      = args.status;
    const unsigned long long lim = args.wait_ns ? args.wait_ns : kDefaultWaitNs;
    constexpr int      kAccStride = BN <= 128 ? 128 : 256;  // TMEM columns between the two accumulators
    constexpr int      kTmemCols  = 2 * kAccStride;         // double-buffered accumulator (a power of two >= 32)
    static_assert(BN % 32 == 0 && BN >= 64 && BN <= 256, "tile width");
    constexpr int      kBNOut    = (EPI == kEpiSwiGLU) ? BN / 2 : BN;

    if (threadIdx.x == 0) {
        *fail_slot = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], A8 ? 1 + kCvtThreads : 1);  // the producer (B bytes) and, for A8, every converter thread
            mbar_init(&empty_bar[s], 1);
            mbar_init(&raw_bar[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tfull_bar[s], 1);
            mbar_init(&tempty_bar[s], 128);
        }
        if (AG)
            for (int s = 0; s < kAgMaxBufs; ++s) mbar_init(&ag_bar[s], 1);
        for (int s = 0; s < kTileRing; ++s) {
            mbar_init(&tr_full[s], 1);
            mbar_init(&tr_empty[s], 1 + 128);
        }
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
            TileWalker walk(args, kBNOut, AROWS);
            TileCoord  tc;
            int        stage = 0;
            uint32_t   phase = 0;
            bool       ok    = true;
            int        ready_group = -1;
            const unsigned long long group_target =
                args.group_ready == nullptr ? 0ull : (args.group_ready_epoch ? *reinterpret_cast<const volatile unsigned long long*>(args.group_ready_epoch) : args.group_ready_target);
            TileFeed feed(args, tile_ring, tr_full, tr_empty);
            bool     ended = false;
            // the tile after the current one, for the weight prefetch (static order: every gridDim-th tile)
            const int  pf_dist = (args.tile_counter == nullptr && args.w_prefetch > 0) ? (args.w_prefetch < kblocks ? args.w_prefetch : kblocks) : 0;
            TileWalker peek(args, kBNOut, AROWS);
            TileCoord  tn;
            // behind the per-group pairs, the trace holds one start time per CTA
            if (args.group_trace != nullptr) args.group_trace[2 * args.num_groups + blockIdx.x] = globaltimer_ns();
            while (ok) {
                const int  lt   = feed.claim(args);
                const bool have = walk.at(lt, tc);
                if (!feed.publish(have ? lt : -1, st, lim)) {
                    ok = false;
                    break;
                }
                if (!have) {
                    ended = true;
                    break;
                }
                if (args.group_ready != nullptr && tc.group != ready_group) {
                    // the rows of this group are written by a kernel that runs beside this one
                    if (args.group_trace != nullptr && blockIdx.x == 0) args.group_trace[2 * tc.group] = globaltimer_ns();
                    if (!wait_flag_ge(args.group_ready + tc.group, group_target, st, 11, tc.group, lim)) {
                        ok = false;
                        break;
                    }
                    if (args.group_trace != nullptr && blockIdx.x == 0) args.group_trace[2 * tc.group + 1] = globaltimer_ns();
                    fence_proxy_async();
                    ready_group = tc.group;
                }
                const CUtensorMap* mapA = &tmA;
                int                arow = tc.row0;
                bool               gate = args.a_ready != nullptr;
                if (AG && args.ag_local_direct && tc.row0 / args.ag_rows == args.ag_rank) {
                    // the own shard is read where it lies: nothing to wait for
                    mapA = &tmAL;
                    arow = tc.row0 - args.ag_rank * args.ag_rows;
                    gate = false;
                }
                if (gate) {
                    // rows [row0, row0+128) must have arrived in local memory
                    const int f0 = tc.row0 / args.a_ready_rows;
                    int       last_row = tc.row0 + kBM - 1;
                    if (last_row >= tc.row_end) last_row = tc.row_end - 1;
                    const int f1 = last_row / args.a_ready_rows;
                    for (int f = f0; f <= f1 && ok; ++f)
                        ok = wait_flag_ge(args.a_ready + f, args.a_ready_target, st, 10, f, lim);
                    if (!ok) break;
                    fence_proxy_async();
                }
                int yb0, yb1;
                if (EPI == kEpiSwiGLU) {
                    yb0 = tc.group * args.rowsB + tc.nt * (BN / 2);
                    yb1 = yb0 + args.N;
                }
                else {
                    yb0 = tc.group * args.rowsB + tc.nt * BN;
                    yb1 = yb0 + BN / 2;
                }
                int  nb0 = 0, nb1 = 0;
                bool have_next = false;
                if (pf_dist) {
                    have_next = peek.at(lt + static_cast<int>(gridDim.x), tn);
                    if (have_next) {
                        if (EPI == kEpiSwiGLU) {
                            nb0 = tn.group * args.rowsB + tn.nt * (BN / 2);
                            nb1 = nb0 + args.N;
                        }
                        else {
                            nb0 = tn.group * args.rowsB + tn.nt * BN;
                            nb1 = nb0 + BN / 2;
                        }
                        have_next = nb0 != yb0;  // the same weight rows again (another row tile of the group): L2 has them
                    }
                }
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (pf_dist) {
                        const int pk = kb + pf_dist;
                        if (pk < kblocks) {
                            tma_prefetch_l2_2d(&tmB, pk * kBK, yb0);
                            tma_prefetch_l2_2d(&tmB, pk * kBK, yb1);
                        }
                        else if (have_next) {
                            tma_prefetch_l2_2d(&tmB, (pk - kblocks) * kBK, nb0);
                            tma_prefetch_l2_2d(&tmB, (pk - kblocks) * kBK, nb1);
                        }
                    }
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, st, 1, stage, lim)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * S::kStageBytes;
                    uint8_t* sb = sa + S::kABytes;
                    if (A8) {
                        mbar_arrive_expect_tx(&raw_bar[stage], S::kRawBytes);
                        tma_load_2d(raw_smem + stage * S::kRawBytes, mapA, &raw_bar[stage], kb * kBK, arow);
                        mbar_arrive_expect_tx(&full_bar[stage], S::kBBytes);
                    }
                    else {
                        mbar_arrive_expect_tx(&full_bar[stage], S::kStageBytes);
                        tma_load_2d(sa, mapA, &full_bar[stage], kb * kBK, arow);
                    }
                    tma_load_2d(sb, &tmB, &full_bar[stage], kb * kBK, yb0);
                    tma_load_2d(sb + S::kBBytes / 2, &tmB, &full_bar[stage], kb * kBK, yb1);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                *fail_slot = 1;
                if (!ended) feed.publish(-1, nullptr, 1000000ull);  // let the roles behind this one leave too
            }
        }
    }
    else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            TileWalker walk(args, kBNOut, AROWS);
            TileCoord  tc;
            int        stage = 0;
            uint32_t   phase = 0;
            int        acc = 0;
            uint32_t   acc_phase = 0;
            bool       ok = true;
            constexpr uint32_t idesc = make_idesc(kFmtBF16, kFmtBF16, kBM, BN);
            TileFeed           feed(args, tile_ring, tr_full, tr_empty);
            while (ok) {
                const int lt = feed.take(st, lim, ok);
                if (lt < 0 || !walk.at(lt, tc)) break;
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
                    for (int k = 0; k < kBK / 16; ++k) {
                        // advance 16 bf16 = 32 bytes along K inside the swizzle row: +2 in the >>4 address field
                        umma_f16(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    }
                    umma_commit(&empty_bar[stage]);  // frees the smem slot when these MMAs retire
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(&tfull_bar[acc]);
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
            if (!ok) *fail_slot = 1;
        }
    }
    else if (A8 && warp >= 6) {
        // ------------------------------ e4m3 -> bf16 expansion of the A tile ------
        const int  r = threadIdx.x - kThreads;  // tile row of this thread
        TileWalker walk(args, kBNOut, AROWS);
        TileCoord  tc;
        int        stage = 0;
        uint32_t   phase = 0;
        bool       ok    = true;
        const int  srow  = args.K / 128;
        while (ok && walk.next(tc)) {
            int grow = tc.row0 + r;  // rows past the end of A read zeros from the TMA fill; their scale must only be addressable
            if (grow >= args.M_total) grow = args.M_total - 1;
            const float* sc_row = args.a_scale + static_cast<long long>(grow) * srow;
            float        sc     = sc_row[0];
            for (int kb = 0; kb < kblocks; ++kb) {
                if ((kb & 1) == 0) sc = sc_row[kb >> 1];  // one scale per 128 elements = two K blocks
                if (!mbar_wait(&raw_bar[stage], phase, st, 5, stage, lim)) {
                    ok = false;
                    break;
                }
                const uint8_t* raw = raw_smem + stage * S::kRawBytes + r * kBK;  // 64 bytes per row, unswizzled
                uint8_t*       dst = smem + stage * S::kStageBytes + r * 128;    // 128 bytes per row, 16-byte chunks XOR-swizzled
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint2 q = *reinterpret_cast<const uint2*>(raw + c * 8);
                    float       v[8];
                    dequant_fp8x8(q, sc, v);
                    *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7)) << 4)) = pack_bf16x8(v);
                }
                fence_proxy_async_smem();  // the tensor core reads this through the async proxy
                mbar_arrive(&full_bar[stage]);
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
        if (!ok) *fail_slot = 1;
    }
    else if (AG && warp >= 6) {
        // ------------------------------ all-gather push ---------------------------
        if (args.ag_src != nullptr && lane == 0) {
            if (!ag_push_bulk(args, ag_bufs, ag_bar, S::kAgBufs, blockIdx.x, gridDim.x, st, lim)) *fail_slot = 1;
        }
    }
    else {
        // ------------------------------ epilogue ----------------------------------
        const int  quad = warp & 3;  // TMEM lane quadrant this warp may access
        TileWalker walk(args, kBNOut, AROWS);
        TileCoord  tc;
        int        acc = 0;
        uint32_t   acc_phase = 0;
        TileFeed   feed(args, tile_ring, tr_full, tr_empty);
        bool       feed_ok = true;
        while (true) {
            const int lt = feed.take(st, lim, feed_ok);
            if (!feed_ok) *fail_slot = 1;
            if (lt < 0 || !walk.at(lt, tc)) break;
            if (!mbar_wait(&tfull_bar[acc], acc_phase, st, 4, acc, lim)) {
                *fail_slot = 1;
                break;
            }
            tc_fence_after_sync();
            const int      row   = tc.row0 + quad * 32 + lane;
            const bool     valid = row < tc.row_end && quad * 32 + lane < AROWS;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kAccStride;
            const int      col0  = tc.nt * kBNOut;

            // Destination of this thread's row (one thread owns one row of the tile).
            unsigned long long drow = 0;  // byte address of column col0 of the row
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
            // Rows leave through shared memory: the thread packs 64 output columns (128 bytes) of its row into its
            // private, padded slot; the warp then writes whole 128-byte lines row by row (see epi_store_piece).
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
                if (cols > kBNOut - c) cols = kBNOut - c;  // tile widths that are not a multiple of 64
                epi_store_piece(my_slot, warp_slots, o, drow + static_cast<unsigned long long>(c) * 2, do_store, cols, lane);
            }
            tc_fence_before_sync();
            mbar_arrive(&tempty_bar[acc]);
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
    }

    // teardown: everyone meets, then the allocating warp frees TMEM
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        if (*fail_slot != 0) {
            // a wait ran out somewhere: give copies still in flight a bounded moment to land
            const unsigned long long t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (args.tile_counter != nullptr && threadIdx.x == 0) {
        // the last CTA to leave puts the scheduler's words back to zero for the next launch (every CTA has taken its
        // final, out-of-range index by now)
        __threadfence();
        if (atomicAdd(args.tile_counter + 1, 1u) == gridDim.x - 1) {
            args.tile_counter[0] = 0;
            args.tile_counter[1] = 0;
            __threadfence();
        }
    }
    // Launched beside the kernel that fills its groups (programmatic dependent launch): do not complete before that
    // kernel has, so that stream order holds for whatever is launched next. A no-op after an ordinary launch.
    if (args.group_ready != nullptr) griddep_wait();
}

}  // namespace gemm
}  // namespace slime
