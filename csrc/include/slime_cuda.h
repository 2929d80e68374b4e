// C API of libslime_cuda.so: every sm_100a kernel launcher and the CUDA-side
// memory plumbing (symmetric heap, IPC import, status pages). All functions
// return 0 on success and a negative value on error; slime_last_error() gives
// the message for the calling thread. `stream` is a cudaStream_t passed as
// void*; `status` is a device (or mapped host) pointer to a 32-byte status page
// or NULL.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

const char* slime_last_error(void);
int         slime_cuda_version(void);

// ---- status pages and small utilities (runtime.cu) -------------------------
// A status page is 32 bytes of mapped pinned host memory: the kernel writes it,
// the host reads it without a copy. *dev_ptr is the address kernels receive.
int slime_status_alloc(void** host_ptr, void** dev_ptr);
int slime_status_free(void* host_ptr);
// Mapped pinned host words usable as flags that a kernel can wait on or set.
int slime_host_flags_alloc(unsigned long long n_words, void** host_ptr, void** dev_ptr);
int slime_host_flags_free(void* host_ptr);
// Test helper: launches one thread that waits (bounded by limit_ns) for *flag >= target.
int slime_wait_flag_kernel(const void* flag, unsigned long long target, unsigned long long limit_ns, void* status,
                           void* stream);
// Writes `value` to the 64-bit word at `flag` with release semantics at system scope, in stream order.
int slime_signal_flag_kernel(void* flag, unsigned long long value, int add, void* stream);

// ---- symmetric heap (symm_heap.cu) ----------------------------------------
// cudaMalloc-backed region with a CUDA IPC handle (64 bytes) that other
// processes on the node can map. Returns the device pointer in *ptr.
int slime_hook_record_value(void* stream, void* dev_word, unsigned long long value);
int slime_hook_wait_mask(void* stream, void* dev_word, unsigned long long mask, unsigned long long limit_ns,
                         void* dev_timeout_word);
int slime_symm_alloc(unsigned long long bytes, void** ptr, unsigned char* ipc_handle_out64);
int slime_symm_free(void* ptr);
int slime_ipc_get_handle(const void* ptr, unsigned char* ipc_handle_out64, unsigned long long* offset_out,
                         unsigned long long* alloc_size_out);
int slime_ipc_open(const unsigned char* ipc_handle64, void** ptr_out);
int slime_ipc_close(void* ptr);
int slime_enable_peer_access(int peer_device);
int slime_memset_async(void* ptr, int value, unsigned long long bytes, void* stream);
int slime_memcpy_async(void* dst, const void* src, unsigned long long bytes, void* stream);

// ---- fp8 block-scaled quantisation (fp8_quant.cu) ---------------------------
int slime_fp8_quant_1x128(const void* x, void* q, float* scales, long long rows, int cols, long long ldx,
                          long long ldq, void* stream);
int slime_fp8_dequant_1x128(const void* q, const float* scales, void* y, long long rows, int cols, long long ldq,
                            long long ldy, void* stream);
int slime_fp8_quant_128x128(const void* w, void* q, float* scales, int rows, int cols, long long ldw, long long ldq,
                            void* stream);

// ---- tcgen05 GEMMs (gemm.cu) -----------------------------------------------
// C[M,N] = A[M,K] * B[N,K]^T, bf16 in, fp32 accumulate, bf16 out.
int slime_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                    long long ldc, void* status, void* stream);
// Same, but a tile of A rows is read only after its arrival flag reached the target
// (a_ready[row / a_ready_rows] >= a_ready_target); m tiles start at m_tile_rotate.
int slime_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, void* status, void* stream);
// CTA pairs with 256 x 512 tiles, tiles ordered in bands of columns that keep their B rows in L2.
int slime_gemm_bf16_wide(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, void* status, void* stream);
int slime_gemm_fp8_blockscaled(const void* Aq, const float* sa, const void* Bq, const float* sb, void* C, int M, int N, int K,
                               long long lda, long long ldb, long long ldc, void* status, void* stream);
int slime_ag_gemm_fp8(int mode, const void* xq_local, const float* sx_local, const void* aq_full, const float* sa_full,
                      const void* Bq, const float* sb, void* C, int rows_local, int N, int K, long long ldb, long long ldc, int rank,
                      int world, const unsigned long long* dst8, const unsigned long long* sdst8, const unsigned long long* flags8,
                      unsigned long long step, int push_blocks, void* status, void* stream);
int slime_grouped_gemm_fp8a(const void* Aq, const float* a_scale, const void* B, void* C, const int* group_offsets, int num_groups,
                            int M_cap, int N, int K, long long lda_bytes, long long ldb, long long ldc, int epilogue, void* status,
                            void* stream);
int slime_gemm_bf16_gated(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, const void* a_ready, int a_ready_rows, unsigned long long a_ready_target,
                          int m_tile_rotate, void* status, void* stream);
// Tensor-parallel all-gather -> GEMM over peer memory; see gemm.cu for the modes.
int slime_ag_gemm(int mode, const void* x_local, const void* a_full, const void* B, void* C, int rows_local, int N,
                  int K, long long ldb, long long ldc, int rank, int world, const unsigned long long* dst8,
                  const unsigned long long* flags8, unsigned long long step, int push_blocks, void* status,
                  void* stream);
// Rows of A are split into num_groups consecutive groups by the device array
// group_offsets[num_groups+1]; group g multiplies B rows [g*rowsB, (g+1)*rowsB).
// epilogue 0: store; 1: SwiGLU (B holds N gate rows then N up rows per group, C is [M,N]);
// 2: scatter row r, scaled by row_scale[r], to scatter_bases8[info >> 48] + (info & 2^48-1) * scatter_row_bytes
//    where info = row_info[r]; the regions may be peer memory; a region >= 8 or slot >= scatter_slots drops the row.
int slime_grouped_gemm_bf16(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                            int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                            const void* row_info, const unsigned long long* scatter_bases8,
                            unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                            const float* row_scale, void* status, void* stream);
// The same on single CTAs with tiles of tile_n = 128, 192, 224 or 256 columns (0 = 256) and the weight boxes asked into
// L2 w_prefetch K blocks (of 64) ahead of the loads (0 = no prefetch); tile_m = 64: row tiles of 64 and a five-stage ring.
int slime_grouped_gemm_bf16_tile(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                 int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                 const void* row_info, const unsigned long long* scatter_bases8,
                                 unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                                 const float* row_scale, int tile_n, int w_prefetch, int tile_m, void* status, void* stream);
// The same on CTA pairs (clusters of two CTAs, 256-row tiles): faster where groups hold several hundred rows or more.
int slime_grouped_gemm_bf16_pair(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                 int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                 const void* row_info, const unsigned long long* scatter_bases8,
                                 unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                                 const float* row_scale, void* status, void* stream);
// The same on CTA pairs with swapped operands (weight rows on the M side of the MMA, a group's tokens on the N side).
int slime_grouped_gemm_bf16_swapped(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                    int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                    const void* row_info, const unsigned long long* scatter_bases8,
                                    unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                                    const float* row_scale, void* status, void* stream);
// The same on CTA pairs with 256 x 512 tiles (two accumulator blocks that share the A tile).
int slime_grouped_gemm_bf16_wide(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                 int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                 const void* row_info, const unsigned long long* scatter_bases8,
                                 unsigned long long scatter_row_bytes, unsigned long long scatter_slots,
                                 const float* row_scale, void* status, void* stream);
// The same GEMM (epilogues 0 and 1) over groups that become readable while it runs: the rows of group g are loaded
// once group_ready[g] (u64, device memory) >= step, step being group_ready_target or *group_ready_epoch when that
// pointer is not null. The kernel that fills the rows must have been launched before this one (another stream).
int slime_grouped_gemm_bf16_gated(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                  int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                  const void* group_ready, unsigned long long group_ready_target,
                                  const void* group_ready_epoch, void* status, void* stream);

// group_trace (u64 [2 * num_groups], device memory, may be null): per group, when CTA 0's producer began to wait for it
// and when it was ready (globaltimer ns). tile_counter (u32 [2], zero before the first launch, may be null): CTAs take
// tiles from a shared counter instead of every gridDim-th tile.
int slime_grouped_gemm_bf16_gated_traced(const void* A, const void* B, void* C, const int* group_offsets, int num_groups,
                                         int M_cap, int N, int K, long long lda, long long ldb, long long ldc, int epilogue,
                                         const void* group_ready, unsigned long long group_ready_target,
                                         const void* group_ready_epoch, void* group_trace, void* tile_counter, void* status,
                                         void* stream);

// ---- expert-parallel dispatch / combine (ep.cu) ------------------------------
// cfg_bytes points at a packed EpConfig (see dlslime_b200/ops/ep.py for the field order).
int slime_ep_config_size(void);
int slime_ep_route(const void* cfg_bytes, const float* logits, int T, int* topk_idx, float* topk_w, int* slot,
                   unsigned int* send_count, unsigned int* block_counter, unsigned long long epoch, int renormalize,
                   void* stream);
int slime_ep_dispatch(const void* cfg_bytes, const void* x, long long ldx, int T, const int* topk_idx, const int* slot,
                      int* group_offsets, unsigned int* block_counter, unsigned long long epoch, int max_blocks,
                      void* status, void* stream);
// Streamed form (rows pushed expert by expert, one arrival word per source rank and local expert, so that the
// receive side and the grouped GEMM start while later experts are still in flight):
//   route_ordered    route + push_off [num_experts + 1]: start of each expert's rows in this rank's push order
//   layout           one block: waits for the counts, writes group_offsets [experts_per_rank + 1]
//   dispatch_ordered permutation + ordered push of rows quantised before with slime_fp8_quant_1x128 (xq, xs dense);
//                    perm [max_tokens * topk], pushed [num_experts] (zeroed scratch)
//   recv_dequant_gated  per local expert: wait for the W arrival words, fp8 -> bf16, publish ready[j] = step;
//                    deq_done [experts_per_rank] zeroed scratch, ready [experts_per_rank] u64
int slime_ep_route_ordered(const void* cfg_bytes, const float* logits, int T, int* topk_idx, float* topk_w, int* slot,
                           unsigned int* send_count, unsigned int* block_counter, unsigned long long epoch, int renormalize,
                           int* push_off, void* stream);
int slime_ep_layout(const void* cfg_bytes, int* group_offsets, unsigned long long epoch, void* status, void* stream);
int slime_ep_dispatch_ordered(const void* cfg_bytes, const void* xq, const float* xs, int T, const int* topk_idx,
                              const int* slot, const int* push_off, int* perm, unsigned int* pushed,
                              unsigned long long epoch, int max_blocks, void* status, void* stream);
int slime_ep_recv_dequant_gated(const void* cfg_bytes, const int* group_offsets, void* y, long long ldy,
                                unsigned int* deq_done, unsigned long long* ready, unsigned long long epoch,
                                int max_blocks, void* status, void* stream);
// permutation + ONE kernel with both roles (two pushing blocks and one receiving block of every three; `blocks` a
// multiple of 3, 0 = three per SM); the gated grouped GEMM launched behind it starts once all its blocks are running
int slime_ep_stream_comm(const void* cfg_bytes, const void* xq, const float* xs, int T, const int* topk_idx, const int* slot,
                         const int* push_off, int* perm, unsigned int* pushed, const int* group_offsets, void* y, long long ldy,
                         unsigned int* deq_done, unsigned long long* ready, unsigned long long* ready_time,
                         unsigned long long epoch, int blocks, void* status, void* stream);
// ready_time (u64 [experts_per_rank], may be null): when each expert's ready word was published (globaltimer ns)
int slime_ep_recv_dequant_gated_traced(const void* cfg_bytes, const int* group_offsets, void* y, long long ldy,
                                       unsigned int* deq_done, unsigned long long* ready, unsigned long long* ready_time,
                                       unsigned long long epoch, int max_blocks, void* status, void* stream);
int slime_ep_recv_dequant(const void* cfg_bytes, const int* group_offsets, void* y, long long ldy, int expected_rows,
                          unsigned long long epoch, void* status, void* stream);
int slime_ep_combine_push(const void* cfg_bytes, const void* y, long long ldy, const int* group_offsets,
                          int expected_rows, void* status, void* stream);
int slime_ep_signal(const void* cfg_bytes, int which, unsigned long long epoch, void* stream);
int slime_ep_wait(const void* cfg_bytes, int which, unsigned long long epoch, void* status, void* stream);
int slime_ep_combine_reduce(const void* cfg_bytes, int T, const int* topk_idx, const float* topk_w, void* out,
                            long long ldo, unsigned long long epoch, int do_signal, void* status, void* stream);
int slime_ep_barrier(const void* cfg_bytes, unsigned long long epoch, void* status, void* stream);

// ---- NVLink endpoint (nvlink_endpoint.cu) -----------------------------------
void* slime_nvlink_ep_create(void);
int   slime_nvlink_ep_destroy(void* ep);
int   slime_nvlink_ep_register(void* ep, unsigned long long addr, unsigned long long length, const char* name);
int   slime_nvlink_ep_unregister(void* ep, int handle);
int   slime_nvlink_ep_local_info(void* ep, int handle, unsigned char* ipc_out64, unsigned long long* offset,
                                 unsigned long long* addr, unsigned long long* length);
int   slime_nvlink_ep_register_remote(void* ep, const char* name, const unsigned char* ipc64, unsigned long long offset,
                                      unsigned long long length, unsigned long long addr, int same_process);
int   slime_nvlink_ep_handle(void* ep, const char* name, int remote);
unsigned long long slime_nvlink_ep_remote_addr(void* ep, int handle);
// out4 = {code, site, block, aux} of the endpoint's kernel status page (code 0 = ok, 402 = a copy never landed, in which
// case the batch's completion word was withheld)
int slime_nvlink_ep_status(void* ep, unsigned int* out4);
int slime_nvlink_ep_status_clear(void* ep);
// process-wide tuning of the batched kernels: work unit in KiB (0 = leave), bulk-copy kernel on / off (negative = leave)
int slime_nvlink_ep_tune(int unit_kb, int bulk);
// tuples: n x {local_handle, remote_handle, remote_offset, local_offset, length} as u64.
int slime_nvlink_ep_transfer(void* ep, const unsigned long long* tuples, int n, int is_write, void* signal,
                             unsigned long long signal_value, int signal_add, int max_blocks, void* stream);

// ---- low-latency all-to-all (alltoall.cu): same configuration bytes as the all-gather -----------------------------
int slime_a2a_push(const void* cfg_bytes, const void* src, unsigned long long row_bytes, int rows_total, int bs, int max_rows,
                   int transpose, const int* offsets, const int* mask, unsigned long long step, unsigned int* block_counter,
                   int do_wait, int max_blocks, void* status, void* stream);
int slime_a2a_wait(const void* cfg_bytes, unsigned long long step, void* status, void* stream);

// One contiguous piece with scalar arguments: a copy-engine (DMA) copy in stream order, then the completion word.
// slime_nvlink_ep_transfer takes the same route by itself for up to four pieces that are one piece or all >= 4 MiB
// (SLIME_NVLINK_NO_COPY_ENGINE in the environment keeps every batch on the kernels).
int slime_nvlink_ep_copy1(void* ep, long long local_handle, long long remote_handle, unsigned long long remote_offset,
                          unsigned long long local_offset, unsigned long long length, int is_write, void* signal,
                          unsigned long long signal_value, void* stream);

// ---- low-latency all-gather (allgather.cu) -----------------------------------
int slime_ag_config_size(void);
int slime_ag_push(const void* cfg_bytes, const void* src, unsigned long long bytes, unsigned long long stride_bytes,
                  unsigned long long step, unsigned int* block_counter, int do_wait, int max_blocks, void* status,
                  void* stream);
int slime_ag_wait(const void* cfg_bytes, unsigned long long step, void* status, void* stream);

// ---- paged KV-cache transfer / pack / unpack (kv_transfer.cu) -----------------
// Moves K and V of one layer for n_tasks pages between a token-major plane pair and a paged plane
// pair (addresses as integers; the paged side may be peer memory). to_paged: token-major -> paged.
// threads per CTA of the transfer kernel for the whole process (32 .. 256, a multiple of 32; default 256)
int slime_kv_tune(int threads);
int slime_kv_transfer(unsigned long long tok_k, unsigned long long tok_v, unsigned long long page_k,
                      unsigned long long page_v, const int* tok_off, const int* blk, const int* ntok, int n_tasks,
                      int page_tokens, unsigned long long row_bytes, unsigned long long tok_rows,
                      unsigned long long page_blocks, int to_paged, void* done_flag, unsigned long long done_value,
                      unsigned int* block_counter, int max_blocks, void* status, void* stream);

#ifdef __cplusplus
}
#endif
