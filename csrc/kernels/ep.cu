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

// ---------------------------------------------------------------------------
// route: one warp per token
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ep_route_kernel(EpConfig cfg, const float* __restrict__ logits, int T,
                                                      int* __restrict__ topk_idx, float* __restrict__ topk_w,
                                                      int* __restrict__ slot, unsigned int* __restrict__ send_count,
                                                      unsigned int* __restrict__ block_counter, unsigned long long epoch,
                                                      int renormalize)
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
    __shared__ bool is_last;
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
            for (int p = 0; p < cfg.world; ++p) {
                unsigned long long* dst = at<unsigned long long>(cfg, p, cfg.off_counts) + cfg.rank * E + e;
                st_release_sys(dst, word);
            }
        }
        if (threadIdx.x == 0) {
            *block_counter = 0;
            // every other CTA has read the old value already (it did so before counting itself in)
            if (cfg.epoch_ptr) *reinterpret_cast<volatile unsigned long long*>(cfg.epoch_ptr) = epoch;
        }
    }
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

int slime_ep_route(const void* cfg_bytes, const float* logits, int T, int* topk_idx, float* topk_w, int* slot,
                   unsigned int* send_count, unsigned int* block_counter, unsigned long long epoch, int renormalize,
                   void* stream)
{
    EpConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (check_cfg(cfg)) return -1;
    if (T < 0 || T > cfg.max_tokens) return fail("ep route: T=%d exceeds max_tokens=%d", T, cfg.max_tokens);
    const int blocks = T > 0 ? (T + 7) / 8 : 1;
    ep_route_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(cfg, logits, T, topk_idx, topk_w, slot,
                                                                          send_count, block_counter, epoch, renormalize);
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
