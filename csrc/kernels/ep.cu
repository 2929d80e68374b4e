// Expert-parallel MoE dispatch and combine over NVLink peer memory.
//
// Every rank owns one symmetric region with the same layout; kernels receive the
// base address of every rank's region (`peers[]`) and write remote memory with
// plain stores. One step is a chain of kernels, each of the form
//     [wait for flags published by earlier kernels]  work  [publish flags]
// so a rank never needs two of its own kernels to run at the same time, and a
// whole multi-rank step can also be replayed rank by rank on a single GPU.
//
//   route      softmax + top-k of the router logits, per-expert send counts and a
//              slot inside each (rank -> expert) stream; the counts row is then
//              broadcast to every rank (one 64-bit word = epoch << 32 | count).
//   dispatch   waits for the W count rows, derives the exact destination row of
//              every (token, expert) pair in the owner's packed buffer, quantises
//              the token to fp8 e4m3 with 1x128 scales once and stores payload,
//              scales and source info straight into the owners' buffers; then
//              publishes "dispatch done" to every rank.
//   (expert FFN: grouped tcgen05 GEMMs; the down projection's epilogue stores
//              each result row into the source rank's combine buffer.)
//   combine    publishes "combine done", waits for the W peers, then reduces the
//              top-k partial rows of every local token with the gate weights.
//
// All waits are bounded and all computed rows are range-checked; problems are
// recorded in the status page and the kernel returns.
#include "common/fp8.cuh"
#include "common/host_utils.h"
#include "common/ptx.cuh"
#include "slime_cuda.h"

using namespace slime;

namespace {

constexpr int kMaxWorld   = 8;
constexpr int kMaxExperts = 256;
constexpr int kMaxTopk    = 8;
constexpr int kChunk      = 512;  // elements one warp moves per step: 16 per lane

struct EpConfig {
    int rank, world, num_experts, experts_per_rank, topk, hidden;
    int max_tokens;  // capacity of the combine buffer in tokens
    int recv_cap;    // capacity of the packed receive buffers in rows
    unsigned long long off_counts;         // u64 [world][num_experts]
    unsigned long long off_dispatch_done;  // u64 [world]
    unsigned long long off_combine_done;   // u64 [world]
    unsigned long long off_barrier;        // u64 [world]
    unsigned long long off_x;              // u8  [recv_cap][hidden]
    unsigned long long off_scale;          // f32 [recv_cap][hidden/128]
    unsigned long long off_info;           // u64 [recv_cap]  (src_rank << 48 | token * topk + k)
    unsigned long long off_combine;        // bf16 [max_tokens * topk][hidden]
    unsigned long long peers[kMaxWorld];   // base address of every rank's region in this rank's address space
    unsigned long long wait_ns;
    // Optional device-resident step counter. When set, the `epoch` argument of every kernel is an offset
    // to *epoch_ptr (route passes 1 and stores the new value when its last CTA finishes, the kernels that
    // follow pass 0), so a whole step can be replayed from a CUDA graph with nothing changing on the host.
    unsigned long long epoch_ptr;
    // Optional trace page (u64 [16][4], device memory; 0 = off). Rows 0..4 belong to the kernels that wait for other
    // ranks {dispatch, receive, combine, wait, barrier}: {calls, start of the last call (globaltimer ns), time the last
    // call waited, total time waited}. Rows 8..15: {rows pushed to peer p so far, calls}. Written by thread 0 of
    // block 0 only; kernels of one buffer run in stream order, so there is nothing to synchronise.
    unsigned long long trace_ptr;
    // Streamed form: u64 [world][experts_per_rank] in the symmetric region. Word (s, j) on rank p holds the last step
    // for which every row of source rank s for p's local expert j has landed.
    unsigned long long off_arrive;
};

enum TraceRow { kTraceDispatch = 0, kTraceReceive = 1, kTraceCombine = 2, kTraceWait = 3, kTraceBarrier = 4, kTracePeers = 8 };

__device__ __forceinline__ bool tracing(const EpConfig& c)
{
    return c.trace_ptr != 0 && blockIdx.x == 0 && threadIdx.x == 0;
}

__device__ __forceinline__ void trace_waited(const EpConfig& c, int row, unsigned long long t0)
{
    unsigned long long*      r   = reinterpret_cast<unsigned long long*>(c.trace_ptr) + 4 * row;
    const unsigned long long dt  = globaltimer_ns() - t0;
    r[0] += 1;
    r[1] = t0;
    r[2] = dt;
    r[3] += dt;
}

__device__ __forceinline__ unsigned long long resolve_epoch(const EpConfig& c, unsigned long long arg)
{
    return c.epoch_ptr ? *reinterpret_cast<const volatile unsigned long long*>(c.epoch_ptr) + arg : arg;
}

template<typename T>
__device__ __forceinline__ T* at(const EpConfig& c, int rank, unsigned long long off)
{
    return reinterpret_cast<T*>(c.peers[rank] + off);
}

// Streamed form: the order in which a rank pushes its rows. Step j of the order covers local expert j of every
// destination, destinations taken round robin starting behind this rank (rank + 1, rank + 2, ..., this rank last), so
// that every rank's expert 0 is complete first, then every rank's expert 1, ...: the order in which the grouped GEMMs
// consume them.
__device__ __forceinline__ int push_order_expert(const EpConfig& c, int o)
{
    const int j = o / c.world;
    const int p = (c.rank + 1 + o % c.world) % c.world;
    return p * c.experts_per_rank + j;
}

// ---------------------------------------------------------------------------
// route: one warp per token
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ep_route_kernel(EpConfig cfg, const float* __restrict__ logits, int T,
                                                      int* __restrict__ topk_idx, float* __restrict__ topk_w,
                                                      int* __restrict__ slot, unsigned int* __restrict__ send_count,
                                                      unsigned int* __restrict__ block_counter, unsigned long long epoch,
                                                      int renormalize, int* __restrict__ push_off)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t    = blockIdx.x * 8 + warp;
    const int E    = cfg.num_experts;
    const int K    = cfg.topk;
    epoch          = resolve_epoch(cfg, epoch);  // read by every CTA before it reports in below
    if (t < T) {
        int   my_e = -1;
        float my_w = 0.f;
        if (logits != nullptr) {
            float v[kMaxExperts / 32];
            float vmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < kMaxExperts / 32; ++j) {
                const int e = lane + 32 * j;
                v[j]        = e < E ? logits[static_cast<long long>(t) * E + e] : -INFINITY;
                vmax        = fmaxf(vmax, v[j]);
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < kMaxExperts / 32; ++j) sum += (lane + 32 * j < E) ? __expf(v[j] - vmax) : 0.f;
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            float sel_sum = 0.f;
            for (int k = 0; k < K; ++k) {
                float bv = -INFINITY;
                int   bi = 0x7fffffff;
#pragma unroll
                for (int j = 0; j < kMaxExperts / 32; ++j) {
                    const int e = lane + 32 * j;
                    if (v[j] > bv || (v[j] == bv && e < bi)) {
                        bv = v[j];
                        bi = e;
                    }
                }
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                    const int   oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (ov > bv || (ov == bv && oi < bi)) {
                        bv = ov;
                        bi = oi;
                    }
                }
#pragma unroll
                for (int j = 0; j < kMaxExperts / 32; ++j)
                    if (lane + 32 * j == bi) v[j] = -INFINITY;
                const float p = __expf(bv - vmax) / sum;
                sel_sum += p;
                if (lane == k) {
                    my_e = bi;
                    my_w = p;
                }
            }
            if (renormalize) my_w /= sel_sum;
            if (lane < K) {
                topk_idx[t * K + lane] = my_e;
                topk_w[t * K + lane]   = my_w;
            }
        }
        else if (lane < K) {
            my_e = topk_idx[t * K + lane];  // routing decided by the caller; negative = skip
        }
        if (lane < K) {
            int s = -1;
            if (my_e >= 0 && my_e < E) s = static_cast<int>(atomicAdd(&send_count[my_e], 1u));
            slot[t * K + lane] = s;
        }
    }
    // last block broadcasts this rank's count row and resets the counters for the next step
    __shared__ bool         is_last;
    __shared__ unsigned int s_cnt[kMaxExperts];
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        is_last = atomicAdd(block_counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (is_last) {
        __threadfence();
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            const unsigned int       cnt  = atomicExch(&send_count[e], 0u);
            const unsigned long long word = (epoch << 32) | cnt;
            s_cnt[e]                      = cnt;
            // The word carries its own step tag and publishes nothing but itself, so a relaxed store is enough. With release
            // semantics every one of the (up to eight) stores of a thread waited for the one before it to be performed
            // at its peer, which made this kernel take 40-50 us on 8 GPUs against 15 us on one.
            for (int p = 0; p < cfg.world; ++p) {
                unsigned long long* dst = at<unsigned long long>(cfg, p, cfg.off_counts) + cfg.rank * E + e;
                st_relaxed_sys(dst, word);
            }
        }
        if (push_off != nullptr) {
            // streamed form: where each expert's rows start in this rank's push order (see push_order_expert)
            __syncthreads();
            if (threadIdx.x == 0) {
                int acc = 0;
                for (int o = 0; o < E; ++o) {
                    const int e = push_order_expert(cfg, o);
                    push_off[e] = acc;
                    acc += static_cast<int>(s_cnt[e]);
                }
                push_off[E] = acc;
            }
        }
        if (threadIdx.x == 0) {
            *block_counter = 0;
            // every other CTA has read the old value already (it did so before counting itself in)
            if (cfg.epoch_ptr) *reinterpret_cast<volatile unsigned long long*>(cfg.epoch_ptr) = epoch;
        }
    }
}

// Streamed form: the (token, k) pairs of this rank listed in push order. perm[push_off[e] + slot] = t * K + k.
__global__ void __launch_bounds__(256) ep_perm_kernel(EpConfig cfg, int T, const int* __restrict__ topk_idx,
                                                     const int* __restrict__ slot, const int* __restrict__ push_off,
                                                     int* __restrict__ perm)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * cfg.topk) return;
    const int e = topk_idx[i], s = slot[i];
    if (e < 0 || e >= cfg.num_experts || s < 0) return;
    perm[push_off[e] + s] = i;
}

// ---------------------------------------------------------------------------
// dispatch: persistent warps over (token, 512-element chunk) units
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpConfig cfg, const __nv_bfloat16* __restrict__ x, long long ldx,
                                                         int T, const int* __restrict__ topk_idx,
                                                         const int* __restrict__ slot, int* __restrict__ group_offsets,
                                                         unsigned int* __restrict__ block_counter,
                                                         unsigned long long epoch, KernelStatus* st)
{
    __shared__ unsigned int s_total[kMaxExperts];
    __shared__ unsigned int s_before[kMaxExperts];  // rows of ranks below mine for this expert
    __shared__ unsigned int s_dst_row[kMaxExperts];
    __shared__ int          s_ok;
    const int E = cfg.num_experts, El = cfg.experts_per_rank, W = cfg.world, K = cfg.topk, H = cfg.hidden;
    const unsigned long long lim = cfg.wait_ns ? cfg.wait_ns : kDefaultWaitNs;

    epoch = resolve_epoch(cfg, epoch);
    if (threadIdx.x == 0) s_ok = 1;
    const unsigned long long trace_t0 = tracing(cfg) ? globaltimer_ns() : 0;
    __syncthreads();
    // 1. wait for the W count rows of this epoch and derive the layout
    const unsigned long long* counts = at<unsigned long long>(cfg, cfg.rank, cfg.off_counts);
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        unsigned int total = 0, before = 0;
        for (int s = 0; s < W; ++s) {
            const unsigned long long* wp = counts + s * E + e;
            unsigned long long        v  = ld_acquire_sys(wp);
            if ((v >> 32) != epoch) {
                const unsigned long long t0 = globaltimer_ns();
                while (((v = ld_acquire_sys(wp)) >> 32) != epoch) {
                    if (globaltimer_ns() - t0 > lim) {
                        report_status(st, K_TIMEOUT, 20, s, epoch, v >> 32);
                        s_ok = 0;
                        break;
                    }
                    __nanosleep(20);
                }
            }
            const unsigned int c = static_cast<unsigned int>(v & 0xffffffffu);
            total += c;
            if (s < cfg.rank) before += c;
        }
        s_total[e]  = total;
        s_before[e] = before;
    }
    __syncthreads();
    if (tracing(cfg)) {
        trace_waited(cfg, kTraceDispatch, trace_t0);
        unsigned long long* peers_row = reinterpret_cast<unsigned long long*>(cfg.trace_ptr) + 4 * kTracePeers;
        for (int p = 0; p < W; ++p) {
            unsigned long long rows = 0;
            for (int e = p * El; e < (p + 1) * El; ++e) rows += counts[cfg.rank * E + e] & 0xffffffffull;
            peers_row[4 * p] += rows;
            peers_row[4 * p + 1] += 1;
        }
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int    first = (e / El) * El;
        unsigned int off   = 0;
        for (int j = first; j < e; ++j) off += s_total[j];
        s_dst_row[e] = off + s_before[e];
        if (blockIdx.x == 0 && e / El == cfg.rank) {
            group_offsets[e - first] = static_cast<int>(min(off, static_cast<unsigned int>(cfg.recv_cap)));
            if (e - first == El - 1)
                group_offsets[El] = static_cast<int>(min(off + s_total[e], static_cast<unsigned int>(cfg.recv_cap)));
        }
    }
    __syncthreads();

    // 2. quantise and push
    if (s_ok) {
        const int       warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int       chunks = H / kChunk;
        const long long units  = static_cast<long long>(T) * chunks;
        const int       gpr    = H / 128;
        for (long long u = static_cast<long long>(blockIdx.x) * 8 + warp; u < units; u += static_cast<long long>(gridDim.x) * 8) {
            const int t = static_cast<int>(u / chunks);
            const int c = static_cast<int>(u - static_cast<long long>(t) * chunks);
            const __nv_bfloat16* src = x + t * ldx + c * kChunk + lane * 16;
            const uint4 r0 = reinterpret_cast<const uint4*>(src)[0];
            const uint4 r1 = reinterpret_cast<const uint4*>(src)[1];
            float       v[16];
            unpack_bf16x8(r0, v);
            unpack_bf16x8(r1, v + 8);
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
            for (int o = 4; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o, 8));
            const Fp8Scale fs    = fp8_scale_from_amax(amax);
            const float    scale = fs.scale;
            const uint2 q0 = quant_fp8x8(v, fs.inv), q1 = quant_fp8x8(v + 8, fs.inv);
            const uint4 q  = make_uint4(q0.x, q0.y, q1.x, q1.y);
            for (int k = 0; k < K; ++k) {
                const int e = topk_idx[t * K + k];
                if (e < 0 || e >= E) continue;
                const unsigned int row = s_dst_row[e] + static_cast<unsigned int>(slot[t * K + k]);
                if (row >= static_cast<unsigned int>(cfg.recv_cap)) {
                    if (lane == 0 && c == 0) report_status(st, K_BAD_INDEX, 21, e, cfg.recv_cap, row);
                    continue;
                }
                const int p = e / El;
                uint8_t*  px = at<uint8_t>(cfg, p, cfg.off_x) + static_cast<unsigned long long>(row) * H + c * kChunk + lane * 16;
                *reinterpret_cast<uint4*>(px) = q;
                if ((lane & 7) == 0)
                    at<float>(cfg, p, cfg.off_scale)[static_cast<unsigned long long>(row) * gpr + c * 4 + (lane >> 3)] = scale;
                if (c == 0 && lane == 0)
                    at<unsigned long long>(cfg, p, cfg.off_info)[row] =
                        (static_cast<unsigned long long>(cfg.rank) << 48) | static_cast<unsigned long long>(t * K + k);
            }
        }
    }
    // 3. the last block to finish tells every rank that this rank's rows have landed
    __shared__ bool is_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        fence_acq_rel_sys();
        is_last = atomicAdd(block_counter, 1u) == gridDim.x - 1;
        fence_acq_rel_sys();
    }
    __syncthreads();
    if (is_last && threadIdx.x < W) {
        fence_acq_rel_sys();
        st_release_sys(at<unsigned long long>(cfg, threadIdx.x, cfg.off_dispatch_done) + cfg.rank, epoch);
        if (threadIdx.x == 0) *block_counter = 0;
    }
}

// ---------------------------------------------------------------------------
// Streamed form of dispatch and receive: the same bytes and the same layout, but pushed expert by expert (in
// push_order_expert order) with one arrival word per (source rank, local expert), so that the receiving rank can
// start on expert 0 while the rows of the later experts are still crossing NVLink. Three kernels that run at the same
// time on three streams: ep_dispatch_ordered_kernel (pushes), ep_recv_dequant_gated_kernel (waits per expert for the
// W arrival words, expands that expert's rows to bf16, then publishes a local "ready" word) and the grouped GEMM,
// whose TMA producer waits for the ready word of a group before it loads that group's first tile. The layer runs the
// first two as ONE kernel (ep_stream_comm_kernel: two pushing blocks and one receiving block per SM) and launches the
// GEMM behind it in the same stream as its programmatic dependent: the GEMM may start once every block of the kernel
// in front of it is running (or done), so a kernel that waits can never keep the kernel it waits for off the device,
// and no second stream (whose work could be queued behind a waiting kernel) is involved. The grids are sized so that
// everything fits on the device together; the GEMM waits for its predecessor's completion at its end. The two roles
// also exist as kernels of their own (ep_dispatch_ordered_kernel, ep_recv_dequant_gated_kernel), launched the
// ordinary way, for callers that replay a group of ranks step by step.
// ---------------------------------------------------------------------------

// Waits for the W count rows of this step; returns false (and reports) when the wait ran out. Fills, per expert,
// the total rows, the rows of lower ranks and this rank's own count.
__device__ __forceinline__ bool ep_wait_counts(const EpConfig& cfg, unsigned long long epoch, KernelStatus* st,
                                               unsigned int* s_total, unsigned int* s_before, unsigned int* s_mine,
                                               int* s_ok)
{
    const int                E = cfg.num_experts, W = cfg.world;
    const unsigned long long lim    = cfg.wait_ns ? cfg.wait_ns : kDefaultWaitNs;
    const unsigned long long* counts = at<unsigned long long>(cfg, cfg.rank, cfg.off_counts);
    if (threadIdx.x == 0) *s_ok = 1;
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        unsigned int total = 0, before = 0, mine = 0;
        for (int s = 0; s < W; ++s) {
            const unsigned long long* wp = counts + s * E + e;
            unsigned long long        v  = ld_acquire_sys(wp);
            if ((v >> 32) != epoch) {
                const unsigned long long t0 = globaltimer_ns();
                while (((v = ld_acquire_sys(wp)) >> 32) != epoch) {
                    if (globaltimer_ns() - t0 > lim) {
                        report_status(st, K_TIMEOUT, 22, s, epoch, v >> 32);
                        *s_ok = 0;
                        break;
                    }
                    __nanosleep(20);
                }
            }
            const unsigned int c = static_cast<unsigned int>(v & 0xffffffffu);
            total += c;
            if (s < cfg.rank) before += c;
            if (s == cfg.rank) mine = c;
        }
        s_total[e]  = total;
        s_before[e] = before;
        if (s_mine) s_mine[e] = mine;
    }
    __syncthreads();
    return *s_ok != 0;
}

// One block: waits for the counts and writes the row prefix of this rank's local experts, so that the kernels that
// walk the groups can be launched without waiting for the dispatch kernel.
__global__ void __launch_bounds__(256) ep_layout_kernel(EpConfig cfg, int* __restrict__ group_offsets,
                                                       unsigned long long epoch, KernelStatus* st)
{
    __shared__ unsigned int s_total[kMaxExperts];
    __shared__ unsigned int s_before[kMaxExperts];
    __shared__ int          s_ok;
    epoch = resolve_epoch(cfg, epoch);
    const bool ok = ep_wait_counts(cfg, epoch, st, s_total, s_before, nullptr, &s_ok);
    if (threadIdx.x == 0) {
        const int    El = cfg.experts_per_rank, first = cfg.rank * El;
        unsigned int off = 0;
        for (int j = 0; j < El; ++j) {
            group_offsets[j] = static_cast<int>(min(off, static_cast<unsigned int>(cfg.recv_cap)));
            off += ok ? s_total[first + j] : 0u;
        }
        group_offsets[El] = static_cast<int>(min(off, static_cast<unsigned int>(cfg.recv_cap)));
    }
}

// One warp per (token, k) pair, in push order. The tokens were quantised once by the stand-alone 1x128 kernel into a
// local staging buffer (xq, xs); the warp copies the token's e4m3 row, its scales and a source word to their exact
// row of the owner's packed buffer with 16-byte loads and stores and nothing else, so that the kernel costs the
// tensor-core kernel it runs beside almost no issue slots. The warp that completes an expert (its pair count reaches
// this rank's count for the expert) publishes the arrival word on the owner.
__device__ __forceinline__ void ep_push_role(const EpConfig& cfg, const uint8_t* __restrict__ xq, const float* __restrict__ xs,
                                             int T, const int* __restrict__ topk_idx, const int* __restrict__ slot,
                                             const int* __restrict__ perm, const int* __restrict__ push_off,
                                             unsigned int* __restrict__ pushed, unsigned long long epoch, KernelStatus* st,
                                             int vb, int nvb)
{
    __shared__ unsigned int s_total[kMaxExperts];
    __shared__ unsigned int s_dst_row[kMaxExperts];  // first the rows of lower ranks, then the destination row
    __shared__ unsigned int s_mine[kMaxExperts];
    __shared__ int          s_ok;
    unsigned int* const     s_before = s_dst_row;
    const int E = cfg.num_experts, El = cfg.experts_per_rank, K = cfg.topk, H = cfg.hidden;
    epoch = resolve_epoch(cfg, epoch);
    const unsigned long long trace_t0 = (cfg.trace_ptr != 0 && vb == 0 && threadIdx.x == 0) ? globaltimer_ns() : 0;
    if (!ep_wait_counts(cfg, epoch, st, s_total, s_before, s_mine, &s_ok)) return;
    if ((cfg.trace_ptr != 0 && vb == 0 && threadIdx.x == 0)) trace_waited(cfg, kTraceDispatch, trace_t0);
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int    first = (e / El) * El;
        unsigned int off   = 0;
        for (int j = first; j < e; ++j) off += s_total[j];
        s_dst_row[e] = off + s_before[e];  // in place: every thread touches only its own experts' entries
        // an expert this rank sends nothing to is complete from this rank's side at once
        if (vb == 0 && s_mine[e] == 0)
            st_release_sys(at<unsigned long long>(cfg, e / El, cfg.off_arrive) + cfg.rank * El + (e - first), epoch);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gpr = H / 128;               // scales per row
    const int row_vecs = H / 16;           // 16-byte pieces of a payload row
    const int scale_vecs = gpr / 4;        // 16-byte pieces of a scale row (hidden is a multiple of 512)
    const int rows = push_off[E];
    for (int r = vb * 8 + warp; r < rows; r += nvb * 8) {
        const int i = perm[r];
        const int e = (i >= 0 && i < T * K) ? topk_idx[i] : -1;
        if (e < 0 || e >= E) {
            if (lane == 0) report_status(st, K_BAD_INDEX, 23, r, T * K, static_cast<unsigned long long>(i));
            continue;
        }
        const int          t   = i / K;
        const unsigned int row = s_dst_row[e] + static_cast<unsigned int>(slot[i]);
        const int          p   = e / El;
        if (row < static_cast<unsigned int>(cfg.recv_cap)) {
            const uint4* src = reinterpret_cast<const uint4*>(xq + static_cast<long long>(t) * H);
            uint4*       dst = reinterpret_cast<uint4*>(at<uint8_t>(cfg, p, cfg.off_x) + static_cast<unsigned long long>(row) * H);
            int v = lane;
            for (; v + 6 * 32 < row_vecs; v += 7 * 32) {
                uint4 tmp[7];
#pragma unroll
                for (int u = 0; u < 7; ++u) tmp[u] = src[v + u * 32];
#pragma unroll
                for (int u = 0; u < 7; ++u) dst[v + u * 32] = tmp[u];
            }
            for (; v < row_vecs; v += 32) dst[v] = src[v];
            if (lane < scale_vecs)
                reinterpret_cast<uint4*>(at<float>(cfg, p, cfg.off_scale) + static_cast<unsigned long long>(row) * gpr)[lane] =
                    reinterpret_cast<const uint4*>(xs + static_cast<long long>(t) * gpr)[lane];
            for (int sv = 32 + lane; sv < scale_vecs; sv += 32)  // rows wider than 16384 elements
                reinterpret_cast<uint4*>(at<float>(cfg, p, cfg.off_scale) + static_cast<unsigned long long>(row) * gpr)[sv] =
                    reinterpret_cast<const uint4*>(xs + static_cast<long long>(t) * gpr)[sv];
            if (lane == 0)
                at<unsigned long long>(cfg, p, cfg.off_info)[row] =
                    (static_cast<unsigned long long>(cfg.rank) << 48) | static_cast<unsigned long long>(i);
        }
        else if (lane == 0) {
            report_status(st, K_BAD_INDEX, 21, e, cfg.recv_cap, row);
        }
        __syncwarp();
        if (lane == 0) {
            fence_acq_rel_sys();  // this row's stores are ordered before the count below, for whoever completes the expert
            if (atomicAdd(&pushed[e], 1u) + 1u == s_mine[e]) {
                atomicExch(&pushed[e], 0u);
                fence_acq_rel_sys();
                st_release_sys(at<unsigned long long>(cfg, p, cfg.off_arrive) + cfg.rank * El + (e - p * El), epoch);
            }
        }
    }
}

__global__ void __launch_bounds__(256, 5) ep_dispatch_ordered_kernel(EpConfig cfg, const uint8_t* __restrict__ xq,
                                                                    const float* __restrict__ xs, int T,
                                                                    const int* __restrict__ topk_idx,
                                                                    const int* __restrict__ slot, const int* __restrict__ perm,
                                                                    const int* __restrict__ push_off,
                                                                    unsigned int* __restrict__ pushed,
                                                                    unsigned long long epoch, KernelStatus* st)
{
    ep_push_role(cfg, xq, xs, T, topk_idx, slot, perm, push_off, pushed, epoch, st, blockIdx.x, gridDim.x);
}

// Receive side of the streamed form. Every block goes through the local experts in order (in small batches): wait
// for the W arrival words of each expert of the batch, expand this block's share of the batch's rows, count itself
// in; the last block publishes ready[j] = step for the batch's experts, which is what the grouped GEMM's producer
// waits for.
__device__ __forceinline__ void ep_recv_role(const EpConfig& cfg, const int* __restrict__ group_offsets,
                                             __nv_bfloat16* __restrict__ y, long long ldy, unsigned int* __restrict__ deq_done,
                                             unsigned long long* __restrict__ ready, unsigned long long* __restrict__ ready_time,
                                             unsigned long long epoch, KernelStatus* st, int vb, int nvb)
{
    __shared__ int s_ok;
    epoch = resolve_epoch(cfg, epoch);
    const int                El = cfg.experts_per_rank, W = cfg.world, gpr = cfg.hidden / 128;
    const unsigned long long lim = cfg.wait_ns ? cfg.wait_ns : kDefaultWaitNs;
    const uint8_t*           q   = at<uint8_t>(cfg, cfg.rank, cfg.off_x);
    const float*             sc  = at<float>(cfg, cfg.rank, cfg.off_scale);
    const unsigned long long* arrive = at<unsigned long long>(cfg, cfg.rank, cfg.off_arrive);
    const unsigned long long trace_t0 = (cfg.trace_ptr != 0 && vb == 0 && threadIdx.x == 0) ? globaltimer_ns() : 0;
    unsigned long long       waited   = 0;
    // Experts are taken in batches of consecutive experts (at most 32 batches per step), so that the fixed cost of a
    // batch (polling the arrival words, the block-wide and grid-wide counting) is paid per ~1/32 of the rows, not per
    // expert: with 256 local experts of ~128 rows each a per-expert round would cost more than the rows themselves.
    const int batch = (El + 31) / 32;
    for (int j0 = 0; j0 < El; j0 += batch) {
        const int j1 = min(El, j0 + batch);
        if (threadIdx.x == 0) s_ok = 1;
        __syncthreads();
        for (int w = threadIdx.x; w < W * (j1 - j0); w += blockDim.x) {
            const int                src = w / (j1 - j0), j = j0 + w % (j1 - j0);
            const unsigned long long w0  = trace_t0 ? globaltimer_ns() : 0;
            if (!wait_flag_ge(arrive + src * El + j, epoch, st, 31, src, lim)) s_ok = 0;
            if (trace_t0 && threadIdx.x == 0) waited += globaltimer_ns() - w0;
        }
        __syncthreads();
        if (!s_ok) break;  // nothing is published for this or any later expert: the GEMM's own wait reports too
        const long long g0 = static_cast<long long>(group_offsets[j0]) * gpr, g1 = static_cast<long long>(group_offsets[j1]) * gpr;
        // four independent 128-element groups per thread and pass: the kernel runs with one block per SM beside the
        // GEMM, so its throughput comes from loads in flight per thread, not from the number of threads
        const long long stride = (static_cast<long long>(nvb) * blockDim.x) >> 4;
        const int       sub    = threadIdx.x & 15;
        for (long long gid = g0 + ((static_cast<long long>(vb) * blockDim.x + threadIdx.x) >> 4); gid < g1; gid += 4 * stride) {
            uint2 raw[4];
            float scl[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long g = gid + u * stride;
                if (g < g1) {
                    raw[u] = *reinterpret_cast<const uint2*>(q + g * 128 + sub * 8);
                    scl[u] = sc[g];
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long g = gid + u * stride;
                if (g < g1) {
                    long long oy = g * 128;
                    if (ldy != cfg.hidden) {
                        const long long row = g / gpr;
                        oy                  = row * ldy + (g - row * gpr) * 128;
                    }
                    float v[8];
                    dequant_fp8x8(raw[u], scl[u], v);
                    *reinterpret_cast<uint4*>(y + oy + sub * 8) = pack_bf16x8(v);
                }
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(&deq_done[j0], 1u) == nvb - 1) {
                atomicExch(&deq_done[j0], 0u);
                __threadfence();
                for (int j = j0; j < j1; ++j) st_release_sys(ready + j, epoch);
                if (ready_time != nullptr) {
                    const unsigned long long now = globaltimer_ns();
                    for (int j = j0; j < j1; ++j) ready_time[j] = now;
                }
            }
        }
    }
    if ((cfg.trace_ptr != 0 && vb == 0 && threadIdx.x == 0)) {
        unsigned long long* r = reinterpret_cast<unsigned long long*>(cfg.trace_ptr) + 4 * kTraceReceive;
        r[0] += 1;
        r[1] = trace_t0;
        r[2] = waited;
        r[3] += waited;
    }
}

__global__ void __launch_bounds__(256) ep_recv_dequant_gated_kernel(EpConfig cfg, const int* __restrict__ group_offsets,
                                                                   __nv_bfloat16* __restrict__ y, long long ldy,
                                                                   unsigned int* __restrict__ deq_done,
                                                                   unsigned long long* __restrict__ ready,
                                                                   unsigned long long* __restrict__ ready_time,
                                                                   unsigned long long epoch, KernelStatus* st)
{
    ep_recv_role(cfg, group_offsets, y, ldy, deq_done, ready, ready_time, epoch, st, blockIdx.x, gridDim.x);
}

// Both roles in ONE kernel, which is what the layer launches: of every three consecutive blocks two push and one
// receives, so that expert 0 is expanded while the later experts are still being pushed, and the grouped GEMM behind
// this kernel is its programmatic dependent: it is scheduled as soon as every block of this kernel is running. (With
// the two roles as two kernels the GEMM, third in the chain, was found to start only when the first kernel had
// completed.) Grid: 3 blocks per SM, all resident beside the GEMM's one CTA per SM.
__global__ void __launch_bounds__(256, 5) ep_stream_comm_kernel(EpConfig cfg, const uint8_t* __restrict__ xq,
                                                               const float* __restrict__ xs, int T,
                                                               const int* __restrict__ topk_idx, const int* __restrict__ slot,
                                                               const int* __restrict__ perm, const int* __restrict__ push_off,
                                                               unsigned int* __restrict__ pushed,
                                                               const int* __restrict__ group_offsets,
                                                               __nv_bfloat16* __restrict__ y, long long ldy,
                                                               unsigned int* __restrict__ deq_done,
                                                               unsigned long long* __restrict__ ready,
                                                               unsigned long long* __restrict__ ready_time,
                                                               unsigned long long epoch, KernelStatus* st)
{
    griddep_launch_dependents();  // this block is running: the grouped GEMM behind this kernel may be scheduled
    const int triple = blockIdx.x / 3, role = blockIdx.x % 3, triples = gridDim.x / 3;  // the grid is a multiple of 3
    if (role == 2)
        ep_recv_role(cfg, group_offsets, y, ldy, deq_done, ready, ready_time, epoch, st, triple, triples);
    else
        ep_push_role(cfg, xq, xs, T, topk_idx, slot, perm, push_off, pushed, epoch, st, 2 * triple + role, 2 * triples);
}

// Waits (bounded) until every rank's flag in `off` reached `epoch`. Called by all threads of a block.
__device__ __forceinline__ bool wait_all_ranks(const EpConfig& cfg, unsigned long long off, unsigned long long epoch,
                                               KernelStatus* st, unsigned int where)
{
    __shared__ int ok;
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    if (threadIdx.x < cfg.world) {
        const unsigned long long lim = cfg.wait_ns ? cfg.wait_ns : kDefaultWaitNs;
        if (!wait_flag_ge(at<unsigned long long>(cfg, cfg.rank, off) + threadIdx.x, epoch, st, where, threadIdx.x, lim)) ok = 0;
    }
    __syncthreads();
    return ok != 0;
}

// ---------------------------------------------------------------------------
// receive side: wait for "dispatch done", then fp8 -> bf16 for the rows that arrived
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ep_recv_dequant_kernel(EpConfig cfg, const int* __restrict__ group_offsets,
                                                             __nv_bfloat16* __restrict__ y, long long ldy,
                                                             unsigned long long epoch, KernelStatus* st)
{
    epoch = resolve_epoch(cfg, epoch);
    const unsigned long long trace_t0 = tracing(cfg) ? globaltimer_ns() : 0;
    if (!wait_all_ranks(cfg, cfg.off_dispatch_done, epoch, st, 30)) return;
    if (tracing(cfg)) trace_waited(cfg, kTraceReceive, trace_t0);
    const int       rows = group_offsets[cfg.experts_per_rank];
    const int       gpr  = cfg.hidden / 128;
    const long long n    = static_cast<long long>(rows) * gpr;
    const uint8_t*  q    = at<uint8_t>(cfg, cfg.rank, cfg.off_x);
    const float*    sc   = at<float>(cfg, cfg.rank, cfg.off_scale);
    for (long long gid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4; gid < n;
         gid += (static_cast<long long>(gridDim.x) * blockDim.x) >> 4) {
        const int sub = threadIdx.x & 15;
        long long oq = gid * 128, oy = gid * 128;  // dense output: a group's offset is its index times 128
        if (ldy != cfg.hidden) {
            const long long row = gid / gpr;
            oy                  = row * ldy + (gid - row * gpr) * 128;
        }
        const uint2 raw = *reinterpret_cast<const uint2*>(q + oq + sub * 8);
        float       v[8];
        dequant_fp8x8(raw, sc[gid], v);
        *reinterpret_cast<uint4*>(y + oy + sub * 8) = pack_bf16x8(v);
    }
}

// ---------------------------------------------------------------------------
// combine, unfused form: copy expert-output rows back to their source ranks
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ep_combine_push_kernel(EpConfig cfg, const __nv_bfloat16* __restrict__ y,
                                                             long long ldy, const int* __restrict__ group_offsets,
                                                             KernelStatus* st)
{
    const int       rows   = group_offsets[cfg.experts_per_rank];
    const int       H      = cfg.hidden;
    const int       chunks = H / 256;  // 256 bf16 = 512 bytes per warp step
    const long long units  = static_cast<long long>(rows) * chunks;
    const int       warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned long long* info = at<unsigned long long>(cfg, cfg.rank, cfg.off_info);
    for (long long u = static_cast<long long>(blockIdx.x) * 8 + warp; u < units; u += static_cast<long long>(gridDim.x) * 8) {
        const int                row = static_cast<int>(u / chunks);
        const int                c   = static_cast<int>(u - static_cast<long long>(row) * chunks);
        const unsigned long long inf = info[row];
        const int                src = static_cast<int>(inf >> 48);
        const unsigned long long s   = inf & 0xffffffffffffull;
        if (src >= cfg.world || s >= static_cast<unsigned long long>(cfg.max_tokens) * cfg.topk) {
            if (lane == 0 && c == 0) report_status(st, K_BAD_INDEX, 40, row, cfg.max_tokens, s);
            continue;
        }
        const uint4 val = *reinterpret_cast<const uint4*>(y + row * ldy + c * 256 + lane * 8);
        *reinterpret_cast<uint4*>(at<__nv_bfloat16>(cfg, src, cfg.off_combine) + s * H + c * 256 + lane * 8) = val;
    }
}

// ---------------------------------------------------------------------------
// combine: publish / wait / gate-weighted reduction of the top-k partial rows
// ---------------------------------------------------------------------------
__global__ void ep_signal_kernel(EpConfig cfg, unsigned long long off, unsigned long long epoch)
{
    epoch = resolve_epoch(cfg, epoch);
    if (threadIdx.x < cfg.world) {
        fence_acq_rel_sys();
        st_release_sys(at<unsigned long long>(cfg, threadIdx.x, off) + cfg.rank, epoch);
    }
}

__global__ void __launch_bounds__(256) ep_combine_reduce_kernel(EpConfig cfg, int T, const int* __restrict__ topk_idx,
                                                               const float* __restrict__ topk_w,
                                                               __nv_bfloat16* __restrict__ out, long long ldo,
                                                               unsigned long long epoch, int do_signal, KernelStatus* st)
{
    epoch = resolve_epoch(cfg, epoch);
    if (do_signal && blockIdx.x == 0 && threadIdx.x < cfg.world) {
        fence_acq_rel_sys();
        st_release_sys(at<unsigned long long>(cfg, threadIdx.x, cfg.off_combine_done) + cfg.rank, epoch);
    }
    const unsigned long long trace_t0 = tracing(cfg) ? globaltimer_ns() : 0;
    if (!wait_all_ranks(cfg, cfg.off_combine_done, epoch, st, 50)) return;
    if (tracing(cfg)) trace_waited(cfg, kTraceCombine, trace_t0);
    const int       H = cfg.hidden, K = cfg.topk;
    const int       chunks = H / 256;
    const unsigned int units = static_cast<unsigned int>(T) * static_cast<unsigned int>(chunks);
    const int          warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const __nv_bfloat16* buf = at<__nv_bfloat16>(cfg, cfg.rank, cfg.off_combine);
    for (unsigned int u = blockIdx.x * 8u + warp; u < units; u += gridDim.x * 8u) {
        const int t = static_cast<int>(u / static_cast<unsigned int>(chunks));
        const int c = static_cast<int>(u - static_cast<unsigned int>(t) * static_cast<unsigned int>(chunks));
        // The row pieces are fetched whether or not their slot is in use (the slot exists in the buffer either way), so
        // that the eight loads do not wait for the index loads; an unused slot is skipped when the sum is formed.
        uint4 part[kMaxTopk];
        int   idx[kMaxTopk];
        float wgt[kMaxTopk];
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k)
            if (k < K) {
                part[k] = *reinterpret_cast<const uint4*>(buf + (static_cast<long long>(t) * K + k) * H + c * 256 + lane * 8);
                idx[k]  = topk_idx[t * K + k];
                wgt[k]  = topk_w[t * K + k];
            }
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k) {
            if (k < K && idx[k] >= 0) {
                float v[8];
                unpack_bf16x8(part[k], v);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = fmaf(wgt[k], v[i], acc[i]);
            }
        }
        *reinterpret_cast<uint4*>(out + t * ldo + c * 256 + lane * 8) = pack_bf16x8(acc);
    }
}

// One small block that waits until every rank's flag reached the step's epoch. Launched in front of a large kernel
// so that the large kernel itself never spins: when two chains of kernels share a GPU (two-batch overlap), a grid of
// spinning blocks can otherwise keep the other chain's signalling block from ever being scheduled.
__global__ void ep_wait_kernel(EpConfig cfg, unsigned long long off, unsigned long long epoch, KernelStatus* st)
{
    epoch = resolve_epoch(cfg, epoch);
    const unsigned long long trace_t0 = tracing(cfg) ? globaltimer_ns() : 0;
    wait_all_ranks(cfg, off, epoch, st, 55);
    if (tracing(cfg)) trace_waited(cfg, kTraceWait, trace_t0);
}

__global__ void ep_barrier_kernel(EpConfig cfg, unsigned long long epoch, KernelStatus* st)
{
    if (threadIdx.x < cfg.world) {
        fence_acq_rel_sys();
        st_release_sys(at<unsigned long long>(cfg, threadIdx.x, cfg.off_barrier) + cfg.rank, epoch);
    }
    const unsigned long long trace_t0 = tracing(cfg) ? globaltimer_ns() : 0;
    wait_all_ranks(cfg, cfg.off_barrier, epoch, st, 60);
    if (tracing(cfg)) trace_waited(cfg, kTraceBarrier, trace_t0);
}

int check_cfg(const EpConfig& c)
{
    if (c.world < 1 || c.world > kMaxWorld) return fail("ep: world size %d not in [1, %d]", c.world, kMaxWorld);
    if (c.rank < 0 || c.rank >= c.world) return fail("ep: bad rank %d", c.rank);
    if (c.num_experts < 1 || c.num_experts > kMaxExperts) return fail("ep: num_experts %d not in [1, %d]", c.num_experts, kMaxExperts);
    if (c.experts_per_rank * c.world != c.num_experts) return fail("ep: experts must divide evenly over ranks");
    if (c.topk < 1 || c.topk > kMaxTopk) return fail("ep: topk %d not in [1, %d]", c.topk, kMaxTopk);
    if (c.hidden <= 0 || c.hidden % kChunk != 0) return fail("ep: hidden (%d) must be a multiple of %d", c.hidden, kChunk);
    for (int i = 0; i < c.world; ++i)
        if (c.peers[i] == 0 || (c.peers[i] & 255) != 0) return fail("ep: peer base %d missing or not 256-byte aligned", i);
    return 0;
}

int grid_for(long long warp_units, int cap_blocks)
{
    long long blocks = (warp_units + 7) / 8;
    if (blocks < 1) blocks = 1;
    if (blocks > cap_blocks) blocks = cap_blocks;
    return static_cast<int>(blocks);
}

}  // namespace

extern "C" {

int slime_ep_config_size(void)
{
    return static_cast<int>(sizeof(EpConfig));
}

static int route_impl(const void* cfg_bytes, const float* logits, int T, int* topk_idx, float* topk_w, int* slot,
                      unsigned int* send_count, unsigned int* block_counter, unsigned long long epoch, int renormalize,
                      int* push_off, void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    if (T < 0 || T > cfg.max_tokens) return fail("ep route: T=%d exceeds max_tokens=%d", T, cfg.max_tokens);
    const int blocks = T > 0 ? (T + 7) / 8 : 1;
    ep_route_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(cfg, logits, T, topk_idx, topk_w, slot,
                                                                          send_count, block_counter, epoch, renormalize,
                                                                          push_off);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_ep_route(const void* cfg_bytes, const float* logits, int T, int* topk_idx, float* topk_w, int* slot,
                   unsigned int* send_count, unsigned int* block_counter, unsigned long long epoch, int renormalize,
                   void* stream)
{
    return route_impl(cfg_bytes, logits, T, topk_idx, topk_w, slot, send_count, block_counter, epoch, renormalize, nullptr, stream);
}

// Streamed form: route that also writes push_off [num_experts + 1], the start of every expert's rows in this rank's
// push order (by expert id; the last entry is the number of (token, k) pairs that go anywhere).
int slime_ep_route_ordered(const void* cfg_bytes, const float* logits, int T, int* topk_idx, float* topk_w, int* slot,
                           unsigned int* send_count, unsigned int* block_counter, unsigned long long epoch, int renormalize,
                           int* push_off, void* stream)
{
    if (push_off == nullptr) return fail("ep route (ordered): push_off is null");
    return route_impl(cfg_bytes, logits, T, topk_idx, topk_w, slot, send_count, block_counter, epoch, renormalize, push_off, stream);
}

int slime_ep_layout(const void* cfg_bytes, int* group_offsets, unsigned long long epoch, void* status, void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    ep_layout_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(cfg, group_offsets, epoch, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

// Streamed dispatch: the permutation kernel followed by the ordered push of rows that were quantised before
// (xq [T, hidden] e4m3 and xs [T, hidden / 128] scales, dense, from slime_fp8_quant_1x128). perm [max_tokens * topk]
// and pushed [num_experts] (zero before the first call; the kernel leaves it zero) are scratch of the caller.
int slime_ep_dispatch_ordered(const void* cfg_bytes, const void* xq, const float* xs, int T, const int* topk_idx,
                              const int* slot, const int* push_off, int* perm, unsigned int* pushed,
                              unsigned long long epoch, int max_blocks, void* status, void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    if (cfg.off_arrive == 0) return fail("ep dispatch (ordered): the buffer has no arrival words");
    if (T < 0 || T > cfg.max_tokens) return fail("ep dispatch: T=%d exceeds max_tokens=%d", T, cfg.max_tokens);
    if ((reinterpret_cast<unsigned long long>(xq) | reinterpret_cast<unsigned long long>(xs)) & 15)
        return fail("ep dispatch (ordered): the staged rows and scales must be 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int    pairs = T * cfg.topk;
    if (pairs > 0) {
        ep_perm_kernel<<<(pairs + 255) / 256, 256, 0, s>>>(cfg, T, topk_idx, slot, push_off, perm);
        SLIME_CUDA_OK(cudaGetLastError());
    }
    const int grid = grid_for(pairs, max_blocks > 0 ? max_blocks : sm_count() * 2);
    ep_dispatch_ordered_kernel<<<grid, 256, 0, s>>>(cfg, static_cast<const uint8_t*>(xq), xs, T, topk_idx, slot, perm,
                                                    push_off, pushed, epoch, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

// Streamed receive: per-expert wait + fp8 -> bf16, publishing ready[j] = step for the grouped GEMM. deq_done
// [experts_per_rank] is zeroed scratch of the caller; ready [experts_per_rank] u64 keeps the last step per expert.
int slime_ep_recv_dequant_gated(const void* cfg_bytes, const int* group_offsets, void* y, long long ldy,
                                unsigned int* deq_done, unsigned long long* ready, unsigned long long epoch,
                                int max_blocks, void* status, void* stream)
{
    return slime_ep_recv_dequant_gated_traced(cfg_bytes, group_offsets, y, ldy, deq_done, ready, nullptr, epoch, max_blocks, status, stream);
}

// The same with a trace: ready_time (u64 [experts_per_rank], device memory, may be null) receives the time
// (globaltimer ns) at which each expert's ready word was published.
int slime_ep_recv_dequant_gated_traced(const void* cfg_bytes, const int* group_offsets, void* y, long long ldy,
                                       unsigned int* deq_done, unsigned long long* ready, unsigned long long* ready_time,
                                       unsigned long long epoch, int max_blocks, void* status, void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    if (cfg.off_arrive == 0) return fail("ep receive (gated): the buffer has no arrival words");
    const int blocks = max_blocks > 0 ? max_blocks : sm_count();
    ep_recv_dequant_gated_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        cfg, group_offsets, static_cast<__nv_bfloat16*>(y), ldy, deq_done, ready, ready_time, epoch, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_ep_dispatch(const void* cfg_bytes, const void* x, long long ldx, int T, const int* topk_idx, const int* slot,
                      int* group_offsets, unsigned int* block_counter, unsigned long long epoch, int max_blocks,
                      void* status, void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    if (T < 0 || T > cfg.max_tokens) return fail("ep dispatch: T=%d exceeds max_tokens=%d", T, cfg.max_tokens);
    if (ldx % 8 != 0) return fail("ep dispatch: ldx must be a multiple of 8 elements");
    const long long units = static_cast<long long>(T) * (cfg.hidden / kChunk);
    const int       grid  = grid_for(units, max_blocks > 0 ? max_blocks : sm_count() * 4);
    ep_dispatch_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        cfg, static_cast<const __nv_bfloat16*>(x), ldx, T, topk_idx, slot, group_offsets, block_counter, epoch,
        static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_ep_recv_dequant(const void* cfg_bytes, const int* group_offsets, void* y, long long ldy, int expected_rows,
                          unsigned long long epoch, void* status, void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    long long threads = static_cast<long long>(expected_rows > 0 ? expected_rows : 1) * (cfg.hidden / 128) * 16;
    long long blocks  = (threads + 255) / 256;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    ep_recv_dequant_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        cfg, group_offsets, static_cast<__nv_bfloat16*>(y), ldy, epoch, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_ep_combine_push(const void* cfg_bytes, const void* y, long long ldy, const int* group_offsets,
                          int expected_rows, void* status, void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    const long long units = static_cast<long long>(expected_rows > 0 ? expected_rows : 1) * (cfg.hidden / 256);
    const int       grid  = grid_for(units, sm_count() * 4);
    ep_combine_push_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        cfg, static_cast<const __nv_bfloat16*>(y), ldy, group_offsets, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_ep_signal(const void* cfg_bytes, int which, unsigned long long epoch, void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    const unsigned long long off = which == 0 ? cfg.off_dispatch_done : which == 1 ? cfg.off_combine_done : cfg.off_barrier;
    ep_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(cfg, off, epoch);
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_ep_wait(const void* cfg_bytes, int which, unsigned long long epoch, void* status, void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    const unsigned long long off = which == 0 ? cfg.off_dispatch_done : which == 1 ? cfg.off_combine_done : cfg.off_barrier;
    ep_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(cfg, off, epoch, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_ep_combine_reduce(const void* cfg_bytes, int T, const int* topk_idx, const float* topk_w, void* out,
                            long long ldo, unsigned long long epoch, int do_signal, void* status, void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    if (T < 0 || T > cfg.max_tokens) return fail("ep combine: T=%d exceeds max_tokens=%d", T, cfg.max_tokens);
    const long long units = static_cast<long long>(T) * (cfg.hidden / 256);
    const int       grid  = grid_for(units, sm_count() * 4);
    ep_combine_reduce_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        cfg, T, topk_idx, topk_w, static_cast<__nv_bfloat16*>(out), ldo, epoch, do_signal,
        static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

// The streamed form as the layer runs it: the permutation kernel, then ONE kernel in which two of every three blocks
// push and the third receives (arguments as for slime_ep_dispatch_ordered and slime_ep_recv_dequant_gated_traced).
// The gated grouped GEMM launched behind it starts as soon as every block of this kernel is running. blocks_per_sm:
// 3 by default (two pushing, one receiving); must be a multiple of 3.
int slime_ep_stream_comm(const void* cfg_bytes, const void* xq, const float* xs, int T, const int* topk_idx, const int* slot,
                         const int* push_off, int* perm, unsigned int* pushed, const int* group_offsets, void* y, long long ldy,
                         unsigned int* deq_done, unsigned long long* ready, unsigned long long* ready_time,
                         unsigned long long epoch, int blocks, void* status, void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    if (cfg.off_arrive == 0) return fail("ep stream comm: the buffer has no arrival words");
    if (T < 0 || T > cfg.max_tokens) return fail("ep stream comm: T=%d exceeds max_tokens=%d", T, cfg.max_tokens);
    if ((reinterpret_cast<unsigned long long>(xq) | reinterpret_cast<unsigned long long>(xs)) & 15)
        return fail("ep stream comm: the staged rows and scales must be 16-byte aligned");
    if (blocks <= 0) blocks = 3 * sm_count();
    if (blocks % 3 != 0) return fail("ep stream comm: the grid (%d) must be a multiple of 3", blocks);
    cudaStream_t s     = static_cast<cudaStream_t>(stream);
    const int    pairs = T * cfg.topk;
    if (pairs > 0) {
        ep_perm_kernel<<<(pairs + 255) / 256, 256, 0, s>>>(cfg, T, topk_idx, slot, push_off, perm);
        SLIME_CUDA_OK(cudaGetLastError());
    }
    // The GEMM that joins this kernel on every SM needs almost all of the SM's shared memory. An SM can only change its
    // split between L1 and shared memory while it is empty, so this kernel asks for the largest shared-memory split
    // itself: the GEMM's CTA then fits beside the resident blocks instead of waiting for them to leave.
    static bool carveout_set[64] = {false};
    SLIME_CUDA_OK(prefer_max_shared_carveout(ep_stream_comm_kernel, carveout_set));
    ep_stream_comm_kernel<<<blocks, 256, 0, s>>>(cfg, static_cast<const uint8_t*>(xq), xs, T, topk_idx, slot, perm, push_off, pushed,
                                                 group_offsets, static_cast<__nv_bfloat16*>(y), ldy, deq_done, ready, ready_time,
                                                 epoch, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_ep_barrier(const void* cfg_bytes, unsigned long long epoch, void* status, void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(cfg, epoch, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

}  // extern "C"
