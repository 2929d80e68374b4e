// Paged KV-cache movement: prefill -> decode page transfer fused with the paged
// scatter, and the local pack / unpack between contiguous and paged layouts.
//
// A KV plane (K or V of one layer) is addressed in two ways:
//   token-major   [tokens][row_bytes]                      (row = all local heads of one token)
//   paged         [blocks][page_tokens][row_bytes]         (block table decides where a page lives)
// A task moves up to page_tokens consecutive rows between "token offset tok_off[p]" on one
// side and "block blk[p]" on the other; the token-major side may itself be a paged cache,
// in which case tok_off = src_block * page_tokens. With to_paged the token-major side is the
// source (pack, or prefill -> decode transfer when the paged side is a peer's cache);
// otherwise the paged side is the source (unpack).
//
// One launch moves K and V of one layer for the whole batch: CTAs walk (task, plane)
// units and copy with 16-byte vectors, eight in flight per thread. The last CTA to finish
// publishes `done_value` at `done_flag` (release, system scope), typically a per-layer
// word in the decode rank's memory, so the consumer can start attention on layer l while
// layer l+1 is still in flight.
#include "common/host_utils.h"
#include "common/ptx.cuh"
#include "slime_cuda.h"

using namespace slime;

namespace {

struct KvArgs {
    unsigned long long tok_k, tok_v;    // token-major planes (base addresses)
    unsigned long long page_k, page_v;  // paged planes (base addresses; may be peer memory)
    const int*         tok_off;         // [n_tasks] first token row of the task on the token-major side
    const int*         blk;             // [n_tasks] block index on the paged side
    const int*         ntok;            // [n_tasks] rows to move (<= page_tokens), or nullptr for full pages
    int                n_tasks;
    int                page_tokens;
    unsigned long long row_bytes;
    unsigned long long tok_rows;     // rows available on the token-major side (range check)
    unsigned long long page_blocks;  // blocks available on the paged side (range check)
    int                to_paged;
    unsigned long long* done_flag;
    unsigned long long  done_value;
    unsigned int*       block_counter;
    KernelStatus*       status;
};

__global__ void __launch_bounds__(256) kv_transfer_kernel(KvArgs a)
{
    const long long units = 2ll * a.n_tasks;
    for (long long u = blockIdx.x; u < units; u += gridDim.x) {
        const int p     = static_cast<int>(u >> 1);
        const int plane = static_cast<int>(u & 1);
        const int toff  = a.tok_off[p];
        const int b     = a.blk[p];
        int       n     = a.ntok ? a.ntok[p] : a.page_tokens;
        if (n > a.page_tokens) n = a.page_tokens;
        if (n <= 0) continue;
        if (toff < 0 || static_cast<unsigned long long>(toff) + n > a.tok_rows || b < 0
            || static_cast<unsigned long long>(b) >= a.page_blocks) {
            if (threadIdx.x == 0) report_status(a.status, K_BAD_INDEX, 80, p, a.page_blocks, static_cast<unsigned long long>(b));
            continue;
        }
        const unsigned long long tok_addr  = (plane ? a.tok_v : a.tok_k) + static_cast<unsigned long long>(toff) * a.row_bytes;
        const unsigned long long page_addr = (plane ? a.page_v : a.page_k)
                                             + static_cast<unsigned long long>(b) * a.page_tokens * a.row_bytes;
        const uint4* src = reinterpret_cast<const uint4*>(a.to_paged ? tok_addr : page_addr);
        uint4*       dst = reinterpret_cast<uint4*>(a.to_paged ? page_addr : tok_addr);
        const unsigned long long nv = static_cast<unsigned long long>(n) * a.row_bytes / 16;
        const unsigned long long nt = blockDim.x;
        unsigned long long       i  = threadIdx.x;
        for (; i + 7ull * nt < nv; i += 8ull * nt) {
            uint4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = src[i + j * nt];
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[i + j * nt] = v[j];
        }
        for (; i < nv; i += nt) dst[i] = src[i];
    }
    if (a.done_flag != nullptr) {
        __shared__ bool is_last;
        __syncthreads();
        if (threadIdx.x == 0) {
            fence_acq_rel_sys();
            is_last = atomicAdd(a.block_counter, 1u) == gridDim.x - 1;
            if (is_last) {
                fence_acq_rel_sys();
                st_release_sys(a.done_flag, a.done_value);
                *a.block_counter = 0;
            }
        }
    }
}

int g_kv_threads = 256;

}  // namespace

extern "C" {

// Threads per CTA of the transfer kernel (32 .. 256, a multiple of 32; default 256) for the whole process. A transfer
// that runs beside a GEMM is best spread thin: one small CTA on every SM slows every GEMM CTA a little, a few large
// CTAs slow a few GEMM CTAs a lot, and the GEMM ends with its slowest CTA.
int slime_kv_tune(int threads)
{
    if (threads < 32 || threads > 256 || threads % 32 != 0) return fail("kv transfer: %d threads per CTA not in [32, 256] or not a multiple of 32", threads);
    g_kv_threads = threads;
    return 0;
}

int slime_kv_transfer(unsigned long long tok_k, unsigned long long tok_v, unsigned long long page_k,
                      unsigned long long page_v, const int* tok_off, const int* blk, const int* ntok, int n_tasks,
                      int page_tokens, unsigned long long row_bytes, unsigned long long tok_rows,
                      unsigned long long page_blocks, int to_paged, void* done_flag, unsigned long long done_value,
                      unsigned int* block_counter, int max_blocks, void* status, void* stream)
{
    if (n_tasks < 0 || page_tokens <= 0) return fail("kv transfer: bad task count or page size");
    if (row_bytes == 0 || row_bytes % 16 != 0) return fail("kv transfer: row_bytes (%llu) must be a positive multiple of 16", row_bytes);
    if (((tok_k | tok_v | page_k | page_v) & 15) != 0) return fail("kv transfer: plane addresses must be 16-byte aligned");
    if (done_flag != nullptr && block_counter == nullptr) return fail("kv transfer: a completion flag needs a block counter");
    KvArgs a{};
    a.tok_k = tok_k, a.tok_v = tok_v, a.page_k = page_k, a.page_v = page_v;
    a.tok_off = tok_off, a.blk = blk, a.ntok = ntok;
    a.n_tasks = n_tasks, a.page_tokens = page_tokens, a.row_bytes = row_bytes;
    a.tok_rows = tok_rows, a.page_blocks = page_blocks, a.to_paged = to_paged;
    a.done_flag     = static_cast<unsigned long long*>(done_flag);
    a.done_value    = done_value;
    a.block_counter = block_counter;
    a.status        = static_cast<KernelStatus*>(status);
    long long grid = 2ll * n_tasks;
    const long long cap = max_blocks > 0 ? max_blocks : sm_count() * 4;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    static bool carveout[64] = {false};  // runs beside the prefill GEMMs: see prefer_max_shared_carveout
    SLIME_CUDA_OK(prefer_max_shared_carveout(kv_transfer_kernel, carveout));
    kv_transfer_kernel<<<static_cast<int>(grid), g_kv_threads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

}  // extern "C"
