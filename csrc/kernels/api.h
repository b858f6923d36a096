// C ABI of the sm_100a kernel library (libnkipy_b200_kernels.so).
// Every entry point takes raw device pointers and a CUDA stream handle, launches
// asynchronously and returns 0 or a negative argument error / positive CUDA
// error code.  Python binds these through ctypes (nkipy_b200/ops/_lib.py).
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace nkb {
int encode_tmap_bf16_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld_elems,
                        uint32_t box_inner, uint32_t box_outer);
int encode_tmap_bf16(CUtensorMap* m, const void* ptr, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                     const uint32_t* box);
int* status_word();
struct GemmArgs;
void mark_bulk(GemmArgs& a);   // gemm_tcgen05.cu: enables the bulk-copy epilogue when the output is 16-byte aligned
int num_sms();
bool pdl_enabled();
}  // namespace nkb

#ifdef __CUDACC__
#include <cuda_runtime.h>
#include <utility>
namespace nkb {
// Launch with the programmatic-stream-serialization attribute (when enabled), so
// the kernel's prologue overlaps the tail of its predecessor in the stream.
template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                      Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return int(cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...));
}
}  // namespace nkb
#endif

extern "C" {
int nkb_init();
// Reads (and optionally clears) the device status word; non-zero = a bounded
// wait inside a kernel gave up (code in the low byte, CTA index above it).
int nkb_status(int reset);
// Enable / disable programmatic dependent launch for all kernels of the library (default on).
void nkb_set_pdl(int enabled);

int nkb_gemm_bf16(const void* A, const void* B, void* out, int rows, int cols, int k, long long lda, long long ldb,
                  long long ldo, int transpose_out, int out_fp32, int splits, long long split_stride, int gated,
                  int gate_off, const void* bias, int bias_on_rows, const void* residual, int block_n, int max_ctas,
                  int weights_operand, int ctas_per_sm, void* stream);
int nkb_gemm_effective_splits(int k, int splits);
int nkb_gemm_bf16_2cta(const void* A, const void* B, void* out, int m, int n, int k, long long lda, long long ldb,
                       long long ldo, const void* bias, const void* residual, int gated, int gate_off, void* stream);
int nkb_gemm_bf16_push(const void* weights, const void* x, int features, int tokens, int k, long long ldw,
                       long long ldx, long long ldo, int splits, const void* bias, int block_n, void* const* peer_out,
                       void* const* peer_flag, int n_peers, int rank, void* done_counter, void* mc_out, void* mc_flag,
                       void* stream);

int nkb_gemm_bf16_grouped(const void* weights, const void* x_sorted, void* out, const int* group_offsets, int num_groups,
                          int features, int k, int total_rows, int max_rows_per_group, long long ldx, long long ldo,
                          int gated, int gate_off, const void* bias, long long bias_group_stride, float act_limit,
                          float act_alpha, int block_n, const int* tile_list, const int* tile_count, int max_tiles,
                          const void* arrive, unsigned int arrive_target, void* stream);
int nkb_moe_dispatch(const int* experts, int tokens, int top_k, int expert_lo, int num_local, const void* x, int hidden,
                     void* x_sorted, int* counts, int* offsets, int* cursors, int* pair_pos, int bn_a, int* tiles_a,
                     int* ntiles_a, int bn_b, int* tiles_b, int* ntiles_b, void* stream);
// expert-parallel token all-to-all (moe_a2a.cu)
int nkb_moe_a2a_dispatch(const void* x, const int* experts, int tokens, int top_k, int hidden, int num_experts,
                         int n_ranks, int rank, unsigned int epoch, void* const* cnt, void* const* cnt_flag,
                         void* const* arrive, void* const* ready, void* const* x_recv, void* const* y, int* cursors,
                         int* sent, int* offsets, int* pair_dest, int capacity_rows, int bn_a, int* tiles_a,
                         int* ntiles_a, int bn_b, int* tiles_b, int* ntiles_b, int* total_rows, void* stream);
int nkb_moe_a2a_combine(const int* pair_dest, const float* weights, int tokens, int top_k, int hidden, int n_ranks,
                        int rank, unsigned int epoch, void* const* cnt, void* const* cnt_flag, void* const* arrive,
                        void* const* ready, void* const* x_recv, void* const* y, void* out, void* stream);
int nkb_moe_combine(const void* y_sorted, const int* pair_pos, const float* weights, int tokens, int top_k, int hidden,
                    void* out, void* stream);

// symmetric memory over CUDA IPC + consumer of the fused GEMM + all-reduce (comm.cu)
int nkb_symm_alloc(void** out, long long bytes);
int nkb_symm_free(void* p);
int nkb_ipc_get_handle(void* p, void* handle_out64);
int nkb_ipc_open(const void* handle64, void** out);
int nkb_ipc_close(void* p);
int nkb_tp_exchange_reduce_rmsnorm(const float* partials, int splits, long long split_stride, const void* y,
                                   void* const* peer_slots, void* const* peer_rowflags, void* mc_slots,
                                   void* mc_rowflags, int n_peers, int rank, const void* local_slots,
                                   const void* local_rowflags, void* seen, void* done_counter,
                                   const void* residual_in, const void* w, void* residual_out, void* normed_out,
                                   int rows, int hidden, float eps, void* stream);
int nkb_tp_reduce_rmsnorm(const void* partials, int slots, const void* flags, int n_src, void* seen,
                          void* done_counter, const void* residual_in, const void* w, void* residual_out,
                          void* normed_out, int rows, int hidden, float eps, void* stream);
int nkb_moe_combine_push(const void* y_sorted, const int* pair_pos, const float* weights, int tokens, int top_k,
                         int hidden, void* const* peer_out, void* const* peer_flag, int n_peers, int rank,
                         void* done_counter, void* mc_out, void* mc_flag, void* stream);
int nkb_argmax_exchange(const float* vals, const int* ids, int rows, int max_rows, int id_offset,
                        void* const* peer_pairs, void* const* peer_flag, int n_peers, int rank, const void* local_pairs,
                        const void* local_flags, void* seen, int* out_ids, void* stream);
// tensor-parallel GEMMs fused with reduce-scatter / all-gather over symmetric memory (gemm_comm.cu)
int nkb_gemm_rs(const void* x, const void* w, void* out, int m, int n, int k, long long ldx, long long ldw,
                long long ldo, void* const* peer_stage, void* const* peer_flags, int flag_stride, int tp, int rank,
                unsigned int epoch, void* stream);
int nkb_ag_gemm(const void* x_local, const void* w, void* out, int m, int n, int k, long long ldx, long long ldw,
                long long ldo, void* const* peer_gather, void* const* peer_flags, int flag_stride, int tp, int rank,
                unsigned int epoch, int comm_ctas, int gated, void* stream);

int nkb_rmsnorm(const void* x, const void* w, void* out, int rows, int hidden, float eps, void* stream);
int nkb_add_rmsnorm(const float* partials, int splits, long long split_stride, const void* x, const void* residual_in,
                    const void* bias, const void* w, void* residual_out, void* normed_out, int rows, int hidden,
                    float eps, void* stream);
int nkb_silu_mul(const void* gate_up, void* out, int rows, int inter, float limit, float alpha, void* stream);
int nkb_silu_mul_partials(const float* partials, int splits, long long stride, const void* bias, void* out, int rows,
                          int inter, float limit, float alpha, void* stream);
int nkb_embedding(const int* ids, const void* table, void* out, int n, int hidden, int vocab, void* stream);
int nkb_rope_kv_append(const void* qkv_bf16, const float* qkv_partials, int splits, long long split_stride,
                       const void* bias, const int* positions, const int* slots, const float* cos_sin,
                       const void* q_norm_w, const void* k_norm_w, float norm_eps, void* q_out, void* k_cache,
                       void* v_cache, int tokens, int nq, int nkv, int head_dim, int max_pos, int block_size,
                       void* stream);
int nkb_decode_advance(int* context_lens, const int* block_table, int* positions, int* slots, int batch, int q_len,
                       int max_blocks, int block_size, void* stream);
int nkb_argmax(const void* logits, int is_fp32, int* out_ids, float* out_vals, int rows, int vocab, long long ld,
               void* stream);
int nkb_sample(const void* logits, int is_fp32, int* out_ids, int rows, int vocab, long long ld, float temperature,
               int top_k, float top_p, unsigned long long seed, unsigned long long step, void* stream);
int nkb_router_topk(const void* logits, int is_fp32, int splits, long long split_stride, const void* bias,
                    float* weights, int* experts, int tokens, int num_experts, int top_k, int mode, void* stream);

int nkb_paged_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                          const int* context_lens, void* out, float* scratch, int batch, int q_len, int nq, int nkv,
                          int head_dim, int block_size, int num_blocks, int max_blocks_per_seq, float scale,
                          int window, const float* sinks, int num_splits, void* stream);
int nkb_paged_attn_decode_fused(const float* qkv_partials, int qkv_splits, long long qkv_split_stride,
                                const void* qkv_bias, const int* positions, const int* slots, const float* cos_sin,
                                const void* q_norm_w, const void* k_norm_w, float norm_eps, int max_pos, void* k_cache,
                                void* v_cache, const int* block_table, const int* context_lens, void* out,
                                float* scratch, int batch, int nq, int nkv, int head_dim, int block_size,
                                int num_blocks, int max_blocks_per_seq, float scale, int window, const float* sinks,
                                int num_splits, void* stream);
long long nkb_paged_attn_decode_scratch_floats(int batch, int q_len, int nq, int head_dim, int num_splits);

int nkb_flash_attn_prefill(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                           const int* q_start, const int* q_lens, const int* context_lens, void* out, int batch,
                           int total_q, int max_q_len, int nq, int nkv, int head_dim, int block_size, int num_blocks,
                           int max_blocks_per_seq, float scale, int causal, int window, const float* sinks,
                           void* stream);
}
