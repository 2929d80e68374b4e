// Low-latency all-gather over NVLink peer memory.
//
// Every rank owns a symmetric buffer  data[2][world][slot_bytes]  and flags
// flags[2][world] (two halves, alternating by step so a fast rank can start step
// n+1 while a slow one still reads the result of step n). A step:
//   push   copy the local contribution into data[half][rank] of EVERY rank (plain
//          16-byte peer stores), then the last CTA publishes flags[half][rank] =
//          step on every rank (release at system scope);
//   wait   block until flags[half][r] >= step for every r (bounded).
// When the buffer lives in a multicast-capable heap (symm_vmm.cu) the push is `multimem.st` to the multicast mapping:
// every 16 bytes and the flag leave the GPU once and the NVSwitch delivers them to all ranks.
// The gathered tensor is data[half] of the local buffer: no extra copy. The issue /
// wait split is the `_hook` form of the reference's removed op
// (AllGatherInterLLBuffer.all_gather_ll / all_gather_ll_hook,
// dlslime/csrc/python/bind.cpp:533-541 in the reference).
#include "common/host_utils.h"
#include "common/ptx.cuh"
#include "slime_cuda.h"

using namespace slime;

namespace {

struct AgConfig {
    int                rank, world;
    unsigned long long off_data;    // u8 [2][world][slot_bytes]
    unsigned long long off_flags;   // u64 [2][world]
    unsigned long long slot_bytes;  // capacity of one rank's contribution
    unsigned long long peers[8];
    unsigned long long wait_ns;
    // Optional device-resident step counter: when set, `step` arguments are offsets to *step_ptr (push passes 1
    // and stores the new value when its last CTA is done, wait passes 0), which makes a call replayable from
    // a CUDA graph.
    unsigned long long step_ptr;
    // Address of the NVLink multicast mapping of the whole region (0 = none). When set, the push is ONE multimem
    // store per 16 bytes, replicated by the switch into every rank's buffer, and the flag one multimem store too.
    unsigned long long mc_base;
};

__global__ void __launch_bounds__(256) ag_push_kernel(AgConfig cfg, const uint4* __restrict__ src, unsigned long long nvec,
                                                     unsigned long long stride_bytes, unsigned long long step,
                                                     unsigned int* block_counter, int do_wait, KernelStatus* st)
{
    if (cfg.step_ptr) step += *reinterpret_cast<const volatile unsigned long long*>(cfg.step_ptr);
    const int                half = static_cast<int>(step & 1);
    const unsigned long long base = cfg.off_data + (static_cast<unsigned long long>(half) * cfg.world) * cfg.slot_bytes
                                    + static_cast<unsigned long long>(cfg.rank) * stride_bytes;
    const unsigned long long tid    = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    if (cfg.mc_base != 0) {
        // four independent loads in flight per thread; each value leaves this GPU once
        uint4* mc = reinterpret_cast<uint4*>(cfg.mc_base + base);
        unsigned long long i = tid;
        for (; i + 3 * stride < nvec; i += 4 * stride) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = src[i + u * stride];
#pragma unroll
            for (int u = 0; u < 4; ++u) multimem_st_v4(mc + i + u * stride, v[u]);
        }
        for (; i < nvec; i += stride) multimem_st_v4(mc + i, src[i]);
    }
    else {
        for (unsigned long long i = tid; i < nvec; i += stride) {
            const uint4 v = src[i];
#pragma unroll 1
            for (int p = 0; p < cfg.world; ++p) reinterpret_cast<uint4*>(cfg.peers[p] + base)[i] = v;
        }
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
    if (cfg.mc_base != 0) {
        if (threadIdx.x == 0) {
            fence_acq_rel_sys();
            multimem_st_release_sys_u64(reinterpret_cast<unsigned long long*>(cfg.mc_base + cfg.off_flags) + half * cfg.world + cfg.rank, step);
            *block_counter = 0;
        }
    }
    else if (threadIdx.x < cfg.world) {
        fence_acq_rel_sys();
        unsigned long long* f = reinterpret_cast<unsigned long long*>(cfg.peers[threadIdx.x] + cfg.off_flags) + half * cfg.world + cfg.rank;
        st_release_sys(f, step);
        if (threadIdx.x == 0) *block_counter = 0;
    }
    if (do_wait && threadIdx.x < cfg.world) {
        const unsigned long long* f = reinterpret_cast<const unsigned long long*>(cfg.peers[cfg.rank] + cfg.off_flags) + half * cfg.world + threadIdx.x;
        wait_flag_ge(f, step, st, 70, threadIdx.x, cfg.wait_ns ? cfg.wait_ns : kDefaultWaitNs);
    }
    // only this CTA is still running, and every CTA read the old value on entry
    if (cfg.step_ptr && threadIdx.x == 0) *reinterpret_cast<volatile unsigned long long*>(cfg.step_ptr) = step;
}

__global__ void ag_wait_kernel(AgConfig cfg, unsigned long long step, KernelStatus* st)
{
    if (cfg.step_ptr) step += *reinterpret_cast<const volatile unsigned long long*>(cfg.step_ptr);
    const int half = static_cast<int>(step & 1);
    if (threadIdx.x < cfg.world) {
        const unsigned long long* f = reinterpret_cast<const unsigned long long*>(cfg.peers[cfg.rank] + cfg.off_flags) + half * cfg.world + threadIdx.x;
        wait_flag_ge(f, step, st, 71, threadIdx.x, cfg.wait_ns ? cfg.wait_ns : kDefaultWaitNs);
    }
}

}  // namespace

extern "C" {

int slime_ag_config_size(void)
{
    return static_cast<int>(sizeof(AgConfig));
}

// Pushes `bytes` (a multiple of 16) from src into slot `rank` of every rank's buffer for `step`
// (steps start at 1 and increase by 1 per call on every rank). stride_bytes is the distance between
// two ranks' contributions in the gathered result (>= bytes, <= slot capacity).
int slime_ag_push(const void* cfg_bytes, const void* src, unsigned long long bytes, unsigned long long stride_bytes,
                  unsigned long long step, unsigned int* block_counter, int do_wait, int max_blocks, void* status,
                  void* stream)
{
    AgConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    if (cfg.world < 1 || cfg.world > 8 || cfg.rank < 0 || cfg.rank >= cfg.world) return fail("all-gather: bad rank/world");
    if (bytes % 16 != 0 || (reinterpret_cast<unsigned long long>(src) & 15) != 0)
        return fail("all-gather: contribution must be 16-byte aligned and a multiple of 16 bytes");
    if (bytes > stride_bytes || stride_bytes > cfg.slot_bytes || stride_bytes % 16 != 0)
        return fail("all-gather: contribution of %llu bytes (stride %llu) exceeds the slot of %llu bytes", bytes, stride_bytes, cfg.slot_bytes);
    const unsigned long long nvec = bytes / 16;
    long long blocks = static_cast<long long>((nvec + 255) / 256);
    const long long cap = max_blocks > 0 ? max_blocks : sm_count() * 2;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    ag_push_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        cfg, static_cast<const uint4*>(src), nvec, stride_bytes, step, block_counter, do_wait, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

int slime_ag_wait(const void* cfg_bytes, unsigned long long step, void* status, void* stream)
{
    AgConfig cfg;
    memcpy(&cfg, cfg_bytes, sizeof(cfg));
    ag_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(cfg, step, static_cast<KernelStatus*>(status));
    SLIME_CUDA_OK(cudaGetLastError());
    return 0;
}

}  // extern "C"
