// Low-latency all-to-all over NVLink peer memory.
//
// Same symmetric layout as the all-gather: data[2][world][slot_bytes] and flags[2][world] on every rank, halves
// alternating by step. Rank r holds rows for every destination; a step stores the rows meant for rank p into slot r of
// p's buffer (plain 16-byte peer stores) and then publishes flags[half][r] = step << 32 | rows on p (release at system
// scope), so the receiver learns how many rows each source sent without a second exchange. Forms:
//   uniform    bs rows per destination; the received tensor is [world * bs, row] ordered by source rank, or, with
//              `transpose`, [bs, world, row] (row b of every source side by side: the sequence <-> head exchange);
//   variable   rows offsets[p] .. offsets[p+1] go to rank p (at most max_rows each); slot s of the receiver holds the
//              rows of source s from its start, the count travels in the flag;
//   mask       destinations with mask[p] == 0 receive no rows (count 0); their flag is still published.
// This is the shape of the reference's removed AllToAllIntraLLBuffer.all_to_all_ll(x, is_transpose, mask, offsets)
// (dlslime/csrc/python/bind.cpp:515-531 in the reference), whose argument meanings are not in that tree.
#include "common/host_utils.h"
#include "common/ptx.cuh"
#include "slime_cuda.h"

using namespace slime;

namespace {

// Field for field the all-gather's configuration (dlslime_b200/ops/allgather.py packs both).
struct A2aConfig {
    int                rank, world;
    unsigned long long off_data;    // u8 [2][world][slot_bytes]
    unsigned long long off_flags;   // u64 [2][world]
    unsigned long long slot_bytes;  // capacity of one source's rows
    unsigned long long peers[8];
    unsigned long long wait_ns;
    unsigned long long step_ptr;    // device-resident step counter (0: `step` is absolute)
};

struct A2aArgs {
    const uint4*       src;        // [rows_total][row_bytes]
    unsigned long long row_bytes;  // multiple of 16
    int                rows_total; // rows of src
    int                bs;         // uniform rows per destination (variable form: unused)
    int                max_rows;   // slot capacity in rows
    int                transpose;  // uniform form only
    const int*         offsets;    // [world + 1] or null
    const int*         mask;       // [world] or null
};

__global__ void __launch_bounds__(256) a2a_push_kernel(A2aConfig cfg, A2aArgs a, unsigned long long step,
                                                      unsigned int* block_counter, int do_wait, KernelStatus* st)
{
    if (cfg.step_ptr) step += *reinterpret_cast<const volatile unsigned long long*>(cfg.step_ptr);
    const int                half = static_cast<int>(step & 1);
    const unsigned long long base = cfg.off_data + (static_cast<unsigned long long>(half) * cfg.world) * cfg.slot_bytes;
    // row ranges per destination, validated once per block
    __shared__ int s_begin[8], s_rows[8];
    if (threadIdx.x < cfg.world) {
        const int p     = threadIdx.x;
        int       begin = a.offsets ? a.offsets[p] : p * a.bs;
        int       rows  = a.offsets ? a.offsets[p + 1] - begin : a.bs;
        if (a.mask && a.mask[p] == 0) rows = 0;
        if (begin < 0 || rows < 0 || rows > a.max_rows || begin + rows > a.rows_total) {
            if (blockIdx.x == 0) report_status(st, K_BAD_INDEX, 80, p, a.max_rows, static_cast<unsigned long long>(static_cast<unsigned int>(rows)));
            rows = 0;
        }
        s_begin[p] = begin;
        s_rows[p]  = rows;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int vpr  = static_cast<int>(a.row_bytes / 16);
    // one warp per 512-byte piece of a row, so that a handful of rows still spreads over many warps; rows are numbered
    // destination by destination
    int total = 0;
    for (int p = 0; p < cfg.world; ++p) total += s_rows[p];
    const unsigned int ppr   = static_cast<unsigned int>((vpr + 31) / 32);
    const unsigned int units = static_cast<unsigned int>(total) * ppr;
    // four pieces per pass: all loads are issued before the first store, so that a warp has 2 KiB in flight
    constexpr int      kPieces = 4;
    const unsigned int stride  = gridDim.x * 8u;
    for (unsigned int u0 = blockIdx.x * 8u + warp; u0 < units; u0 += stride * kPieces) {
        uint4  x[kPieces];
        uint4* to[kPieces];
#pragma unroll
        for (int j = 0; j < kPieces; ++j) {
            const unsigned int u = u0 + j * stride;
            to[j]                = nullptr;
            if (u < units) {
                const unsigned int w = u / ppr;
                const int          v = static_cast<int>(u - w * ppr) * 32 + lane;
                int                p = 0, b = static_cast<int>(w);
                while (b >= s_rows[p]) b -= s_rows[p++];  // at most world - 1 steps
                unsigned long long out_row;
                if (a.offsets)
                    out_row = static_cast<unsigned long long>(cfg.rank) * a.max_rows + b;
                else if (a.transpose)
                    out_row = static_cast<unsigned long long>(b) * cfg.world + cfg.rank;
                else
                    out_row = static_cast<unsigned long long>(cfg.rank) * a.bs + b;
                if (v < vpr) {
                    x[j]  = a.src[static_cast<unsigned long long>(s_begin[p] + b) * vpr + v];
                    to[j] = reinterpret_cast<uint4*>(cfg.peers[p] + base + out_row * a.row_bytes) + v;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kPieces; ++j)
            if (to[j]) *to[j] = x[j];
    }
    __shared__ bool is_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        fence_acq_rel_sys();
        is_last = atomicAdd(block_counter, 1u) == gridDim.x - 1;
        fence_acq_rel_sys();
    }
    __syncthreads();
    if (!is_last) return;
    if (threadIdx.x < cfg.world) {
        fence_acq_rel_sys();
        unsigned long long* f = reinterpret_cast<unsigned long long*>(cfg.peers[threadIdx.x] + cfg.off_flags) + half * cfg.world + cfg.rank;
        st_release_sys(f, (step << 32) | static_cast<unsigned long long>(s_rows[threadIdx.x]));
        if (threadIdx.x == 0) *block_counter = 0;
    }
    if (do_wait && threadIdx.x < cfg.world) {
        const unsigned long long* f = reinterpret_cast<const unsigned long long*>(cfg.peers[cfg.rank] + cfg.off_flags) + half * cfg.world + threadIdx.x;
        wait_flag_ge(f, step << 32, st, 81, threadIdx.x, cfg.wait_ns ? cfg.wait_ns : kDefaultWaitNs);
    }
    // only this CTA is still running, and every CTA read the old value on entry
    if (cfg.step_ptr && threadIdx.x == 0) *reinterpret_cast<volatile unsigned long long*>(cfg.step_ptr) = step;
}

__global__ void a2a_wait_kernel(A2aConfig cfg, unsigned long long step, KernelStatus* st)
{
    if (cfg.step_ptr) step += *reinterpret_cast<const volatile unsigned long long*>(cfg.step_ptr);
    const int half = static_cast<int>(step & 1);
    if (threadIdx.x < cfg.world) {
        const unsigned long long* f = reinterpret_cast<const unsigned long long*>(cfg.peers[cfg.rank] + cfg.off_flags) + half * cfg.world + threadIdx.x;
        wait_flag_ge(f, step << 32, st, 82, threadIdx.x, cfg.wait_ns ? cfg.wait_ns : kDefaultWaitNs);
    }
}

}  // namespace

extern "C" {

// Sends rows of `src` ([rows_total, row_bytes], 16-byte aligned, row_bytes a multiple of 16) to every rank for `step`
// (steps start at 1 and increase by 1 per call on every rank; below 2^31). Uniform form: offsets == null and
// rows_total == world * bs. Variable form: offsets = int32 [world + 1] on the device. mask = int32 [world] on the
// device or null. max_rows * row_bytes must fit the slot.
int slime_a2a_push(const void* cfg_bytes, const void* src, unsigned long long row_bytes, int rows_total, int bs, int max_rows,
                   int transpose, const int* offsets, const int* mask, unsigned long long step, unsigned int* block_counter,
                   int do_wait, int max_blocks, void* status, void* stream)
{
    A2aConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (cfg.world < 1 || cfg.world > 8 || cfg.rank < 0 || cfg.rank >= cfg.world) return fail("all-to-all: bad rank/world");
    if (row_bytes == 0 || row_bytes % 16 != 0 || (reinterpret_cast<unsigned long long>(src) & 15) != 0)
        return fail("all-to-all: rows must be 16-byte aligned and a multiple of 16 bytes long");
    if (rows_total < 0 || max_rows < 0 || static_cast<unsigned long long>(max_rows) * row_bytes > cfg.slot_bytes)
        return fail("all-to-all: %d rows of %llu bytes exceed the slot of %llu bytes", max_rows, row_bytes, cfg.slot_bytes);
    if (!offsets) {
        if (bs < 0 || bs > max_rows || static_cast<long long>(bs) * cfg.world != rows_total)
            return fail("all-to-all: uniform form needs world * bs == rows (bs=%d, world=%d, rows=%d, max %d)", bs, cfg.world,
                        rows_total, max_rows);
    }
    else if (transpose) {
        return fail("all-to-all: the transposed layout exists only for the uniform form");
    }
    A2aArgs a{static_cast<const uint4*>(src), row_bytes, rows_total, bs, max_rows, transpose, offsets, mask};
    const long long pieces = static_cast<long long>(rows_total) * static_cast<long long>((row_bytes / 16 + 31) / 32);
    if (pieces >= (1ll << 32)) return fail("all-to-all: %d rows of %llu bytes are more than one launch moves", rows_total, row_bytes);
    long long blocks = (pieces + 7) / 8;
    const long long cap = max_blocks > 0 ? max_blocks : sm_count() * 2;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    a2a_push_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        cfg, a, step, block_counter, do_wait, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_a2a_wait(const void* cfg_bytes, unsigned long long step, void* status, void* stream)
{
    A2aConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    a2a_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(cfg, step, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

}  // extern "C"
