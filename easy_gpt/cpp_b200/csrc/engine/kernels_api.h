// The C interface of the kernel library (libeasygpt_kernels: the hand-written sm_100a kernels of this folder), as the
// native engine calls it.  Every launcher takes raw device pointers and a stream, returns the launch's cudaError_t
// as an int (cudaErrorInvalidValue also when it refuses a size it does not take) and allocates nothing.
// (tests/test_native_build.py compares this file with the launchers' definitions.)
#pragma once
#include <cuda_runtime.h>

extern "C" {
// activation.cu
int eg_swiglu(cudaStream_t stream, int dtype, const void* gate_up, int ld, void* out, int ldo, int tokens, int inter);
// attention_generic.cu
int eg_attention_generic(cudaStream_t stream, int dtype, const void* q, int ldq, const void* k_cache, const void* v_cache, const int* block_table, int table_stride, const int* token_seq, const int* positions, void* out, int ldo, int tokens, int num_heads, int num_kv_heads, int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages, int window, float scale, int* status);
// attention_paged.cu
int eg_attention_paged(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache, const int* block_table, int table_stride, const int* token_seq, const int* positions, const int* seq_context, void* out, int ldo, float* partial_acc, float* partial_ml, int tokens, int num_heads, int num_kv_heads, int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages, int window, float scale, int splits, int* status, const void* prefetch, long long prefetch_bytes, int* counters, int use_pdl, unsigned long long* trace, const int* token_list);
// attention_paged.cu
int eg_attention_prefill(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache, const int* block_table, int table_stride, const int* positions, const int* tiles, int num_tiles, void* out, int ldo, int num_heads, int num_kv_heads, int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages, int window, float scale, int* status);
// attention_tcgen05.cu
int eg_attention_prefill_tcgen05(cudaStream_t stream, const void* q, long long ldq, int total_tokens, const void* k_cache, const void* v_cache, const int* block_table, int table_stride, const int* positions, const int* tiles, int num_tiles, void* out, long long ldo, int num_heads, int num_kv_heads, int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages, int window, float scale, int* status, long long* trace, int max_parts, int part_tiles, float* partial_o, float* partial_ml, int* queue);
int eg_attention_prefill_groups(int head_dim);
// embedding.cu
int eg_embedding_gather(cudaStream_t stream, int dtype, const int* ids, const void* table, float* residual, int tokens, int hidden, int vocab, int* status);
// engine_ops.cu
int eg_add_into_f32(cudaStream_t stream, float* residual, const void* delta, int delta_dtype, long long n);
// engine_ops.cu
int eg_convert_rows(cudaStream_t stream, const void* src, int src_dtype, void* dst, int dst_dtype, long long n);
// gemm_f32.cu
int eg_gemm_f32_nt(cudaStream_t stream, const float* A, int lda, const float* W, int ldw, const float* bias, float* C, int ldc, int M, int N, int K);
// gemm_skinny.cu
int eg_gemm_skinny(cudaStream_t stream, int epilogue, int norm, int use_pdl, const void* W, long long ldw, const float* bias, int M, int N, int K, const void* x, long long ldx, const float* resid_in, float* resid_out, const void* delta, const float* gain, float eps, void* out, long long ldo, int row_blocks, int k_slices, int k_split, float* scratch, int* counters, int num_heads, int num_kv_heads, int head_dim, const int* positions, const int* slot_map, void* k_cache, void* v_cache, const float* inv_freq, int page_size, long long page_stride, long long head_stride, long long pool_slots, int* status, const void* prefetch, long long prefetch_bytes, unsigned long long* trace, const float* ss_in, int ss_parts, float* resid_inout, const float* gain_out, void* xn_out, float* ss_out);
// gemm_tcgen05.cu
int eg_gemm_tcgen05(cudaStream_t stream, int epilogue, const void* A, long long lda, const void* W, long long ldw, const float* bias, void* out, long long ldo, int M, int N, int K, int* status);
// gemm_tcgen05.cu
int eg_gemm_tcgen05_pair(cudaStream_t stream, int epilogue, const void* A, long long lda, const void* W, long long ldw, const float* bias, void* out, long long ldo, int M, int N, int K, int tile_n, int* status, long long* trace);
// norm.cu
int eg_add_rmsnorm(cudaStream_t stream, int delta_dtype, int out_dtype, float* residual, const void* delta, const int* rows, const float* gain, void* out, int num_rows, int hidden, float eps);
// rope_cache.cu
int eg_rope_table(cudaStream_t stream, const int* positions, const float* inv_freq, float* table, int tokens, int half);
// rope_cache.cu
int eg_rope_cache_vec(cudaStream_t stream, int dtype, void* qkv, int ld, const float* table, const int* slot_map, void* k_cache, void* v_cache, int tokens, int num_heads, int num_kv_heads, int head_dim, int page_size, long long page_stride, long long head_stride, long long pool_slots, int* status);
// rope_cache.cu
int eg_rope_cache(cudaStream_t stream, int dtype, void* qkv, int ld, const float* bias, const int* positions, const int* slot_map, void* k_cache, void* v_cache, const float* inv_freq, int tokens, int num_heads, int num_kv_heads, int head_dim, int rotary_dim, int page_size, long long page_stride, long long head_stride, long long pool_slots, int* status);
// sampling.cu
int eg_argmax(cudaStream_t stream, const float* logits, long long ld, int rows, int vocab, int* out, int blocks_per_row, float* part_val, int* part_idx, int* counters);
// sampling.cu
int eg_sample(cudaStream_t stream, const float* logits, long long ld, int rows, int vocab, const float* temperature, const int* top_k, const float* top_p, const float* uniform, int* out);
// decode_fused.cu
int eg_decode_fused_smem(int stages, int xs_bytes, int num_ops, int num_tmpls);
// decode_fused.cu
int eg_decode_fused(cudaStream_t stream, const void* tmpls, int num_tmpls, const void* ops, int num_ops, int tokens, int stages, int xs_bytes, int ctas, unsigned* sync, int* status, unsigned long long* trace);
// layernorm.cu
int eg_add_layernorm(cudaStream_t stream, float* residual, const void* delta_a, int dtype_a, const void* delta_b, int dtype_b, const int* rows, const float* gain1, const float* bias1, void* out1, const float* gain2, const float* bias2, void* out2, int out_dtype, int num_rows, int hidden, float eps);
// engine_ops.cu
int eg_stream_add(cudaStream_t stream, float* residual, const float* first, const float* offset, int tokens, int hidden);
// engine_ops.cu
int eg_softcap(cudaStream_t stream, float* x, long long n, float cap);
// selective_scan.cu
int eg_conv_silu(cudaStream_t stream, int dtype, const void* x, long long ldx, const float* conv_w, const float* conv_b, const float* state, long long slot_floats, const int* token_seq, const int* seq_starts, const int* seq_slots, void* u, long long ldu, int tokens, int channels, int taps);
// selective_scan.cu
int eg_conv_state(cudaStream_t stream, int dtype, const void* x, long long ldx, float* state, long long slot_floats, const int* seq_starts, const int* seq_slots, int num_seqs, int channels, int taps);
// selective_scan.cu
int eg_step_sizes(cudaStream_t stream, const float* low, long long ldl, const float* dw, const float* db, float* dt, int tokens, int channels, int rank);
// selective_scan.cu
int eg_selective_scan(cudaStream_t stream, int dtype, const void* u, long long ldu, const float* dt, const float* dt_bias, const float* low, long long ldl, int b_col, int c_col, const float* A, const float* D, const void* z, long long ldz, float* state, long long slot_floats, long long state_offset, const int* seq_starts, const int* seq_slots, void* y, long long ldy, int num_seqs, int channels, int states, int states_per_lane);
// attention_latent.cu
int eg_latent_prepare(cudaStream_t stream, const float* down, long long ld, int q_rank, int rank, int rot, int rot_dims, const float* gain_q, const float* gain_c, float eps, const float* inv_freq, const int* positions, const int* slot_map, void* cache, int cache_dtype, int page_size, long long page_stride, long long pool_slots, void* cq, int cq_dtype, int tokens, int* status);
// attention_latent.cu
int eg_latent_absorb(cudaStream_t stream, int w_dtype, const float* q, long long ldq, const void* Uk, const int* positions, const float* inv_freq, int rot_dims, float scale, float* qa, int tokens, int heads, int dim, int rot, int rank);
// attention_latent.cu
int eg_attention_latent(cudaStream_t stream, int cache_dtype, const float* qa, const void* cache, const int* block_table, int table_stride, const int* token_seq, const int* positions, const float* sink, float* out, int tokens, int heads, int rank, int rot, int page_size, long long page_stride, int num_pages, int* status);
// attention_latent.cu
int eg_latent_expand(cudaStream_t stream, int w_dtype, const float* o, const void* Uv, void* out, int out_dtype, long long ldo, int tokens, int heads, int vdim, int rank);
// moe.cu
int eg_moe_route(cudaStream_t stream, int dtype, const void* h, long long ld, const float* router, const float* correction, const float* gate_w, float* logits, int* ids, float* weights, float* gate, int tokens, int width, int outputs, int top, int scoring);
// moe.cu
int eg_moe_hidden(cudaStream_t stream, int dtype, const void* h, long long ld, const void* gate_up, const int* ids, const float* input_weights, void* act, int tokens, int width, int ff, int top, int experts, int activation, float limit);
// moe.cu
int eg_moe_combine(cudaStream_t stream, int dtype, const void* h, long long ld, const void* act, const void* down, const int* ids, const float* weights, const void* shared, int shared_dtype, const float* gate, float* out, int tokens, int width, int ff, int top, int experts);
// moe.cu
int eg_moe_dispatch(cudaStream_t stream, const void* h, long long ld, const int* ids, const float* input_weights, int* counts, int* starts, int* cursors, int* tile_group, int* row_of, void* rows, int tokens, int width, int top, int experts, int max_rows);
// moe.cu
int eg_moe_gather(cudaStream_t stream, const void* y, const int* row_of, const int* ids, const float* weights, const void* h, long long ld, const void* shared, int shared_dtype, const float* gate, float* out, int tokens, int width, int top, int experts);
// gemm_tcgen05.cu
int eg_gemm_tcgen05_grouped(cudaStream_t stream, int epilogue, const void* A, long long lda, const void* W, long long ldw, void* out, long long ldo, int max_rows, int N, int K, int groups, const int* tile_group, int* status);
// gemm_tcgen05.cu
int eg_gemm_tcgen05_few(cudaStream_t stream, int epilogue, int use_pdl, const void* A, long long lda, const void* W, long long ldw, const float* bias, void* out, long long ldo, int M, int N, int K, int tile_n, int slices, float* partial, int* tickets, int* status);
// attention_latent_mma.cu
int eg_attention_latent_mma_takes(int rank, int rot);
// attention_latent_mma.cu
int eg_attention_latent_mma(cudaStream_t stream, const void* qa, const void* cache, const int* block_table, int table_stride, const int* token_seq, const int* positions, const float* sink, void* out, float* part_o, float* part_ml, int tokens, int heads, int rank, int rot, int page_size, long long page_stride, int num_pages, int splits, int* status);
// attention_latent_mma.cu
int eg_latent_rotate_query(cudaStream_t stream, const void* q, long long ldq, const int* positions, const float* inv_freq, int rot_dims, float scale, void* qa, int tokens, int heads, int dim, int rot, int rank);
// sandwich.cu
int eg_token_shift(cudaStream_t stream, const float* rows, const float* mu, float* state, long long slot_floats, const int* token_seq, const int* seq_starts, const int* seq_slots, void* out, int out_dtype, int tokens, int hidden);
// sandwich.cu
int eg_rmsnorm_shift(cudaStream_t stream, const float* residual, const float* gain, float eps, const float* mu, float* state, long long slot_floats, const int* token_seq, const int* seq_starts, const int* seq_slots, void* out, int out_dtype, int tokens, int hidden);
// sandwich.cu
int eg_rmsnorm_add(cudaStream_t stream, float* residual, const void* y, int y_dtype, long long ldy, const float* gain, float eps, int tokens, int hidden);
// sandwich.cu
int eg_rmsnorm_add_norm(cudaStream_t stream, float* residual, const void* y, int y_dtype, long long ldy, const float* gain, float eps, const float* gain2, float eps2, void* out, int out_dtype, int tokens, int hidden);
// sandwich.cu
int eg_xielu(cudaStream_t stream, const void* x, int x_dtype, long long ldx, void* out, int out_dtype, long long ldo, int tokens, int n, float ap, float an);
// sandwich.cu
int eg_embedding_gather_scaled(cudaStream_t stream, int dtype, const int* ids, const void* table, float* residual, int tokens, int hidden, int vocab, float scale, int* status);
// sandwich.cu
int eg_scale_f32(cudaStream_t stream, float* x, long long n, float s);
// attention_sink.cu
int eg_sink_attention_prepare(cudaStream_t stream, int dtype, const float* proj, long long ld, const float* table, int rot_dims, float magnitude, const int* slot_map, void* k_cache, void* v_cache, int row_stride, long long head_stride, int page_size, long long page_stride, long long pool_slots, void* q_out, int tokens, int heads, int kv_heads, int dk, int dv, float unit_eps, int* status);
// attention_sink.cu
int eg_sink_attention(cudaStream_t stream, int dtype, const void* q, const void* k_cache, const void* v_cache, int row_stride, long long head_stride, const int* block_table, int table_stride, const int* token_seq, const int* positions, const int* token_list, void* out, long long ldo, int num_tokens, int heads, int kv_heads, int dk, int dv, int page_size, long long page_stride, int num_pages, int window, float scale, int has_sink, float sink_logit, int* status);
// attention_paged.cu
int eg_attention_paged_sink(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache, const int* block_table, int table_stride, const int* token_seq, const int* positions, const int* seq_context, void* out, int ldo, float* partial_acc, float* partial_ml, int tokens, int num_heads, int num_kv_heads, int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages, int window, float scale, int splits, int* status, int* counters, int use_pdl, const int* token_list, float sink_logit);
// attention_paged.cu
int eg_attention_prefill_sink(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache, const int* block_table, int table_stride, const int* positions, const int* tiles, int num_tiles, void* out, int ldo, int num_heads, int num_kv_heads, int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages, int window, float scale, int* status, float sink_logit);
// attention_tcgen05.cu
int eg_attention_prefill_tcgen05_sink(cudaStream_t stream, const void* q, long long ldq, int total_tokens, const void* k_cache, const void* v_cache, const int* block_table, int table_stride, const int* positions, const int* tiles, int num_tiles, void* out, long long ldo, int num_heads, int num_kv_heads, int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages, int window, float scale, int* status, int max_parts, int part_tiles, float* partial_o, float* partial_ml, int* queue, float sink_logit);
// gemm_tcgen05.cu
int eg_gemm_tcgen05_pair_xielu(cudaStream_t stream, const void* A, long long lda, const void* W, long long ldw, void* out, long long ldo, int M, int N, int K, int tile_n, int* status, float act_a, float act_b);
// gemm_skinny.cu
int eg_gemm_skinny_xielu(cudaStream_t stream, int use_pdl, const void* W, long long ldw, int M, int N, int K, const void* x, long long ldx, void* out, long long ldo, int row_blocks, int k_slices, int k_split, float* scratch, int* counters, int* status, float act_a, float act_b);
// gated_delta.cu
int eg_gated_delta_plan(int dk, int dv, int* rows_per_lane, int* lanes);
// gated_delta.cu
int eg_gated_delta(cudaStream_t stream, float* qkv, long long ldq, int q_col, int k_col, int v_col, const float* proj, long long ldp, int b_col, int a_col, int z_col, const float* a_log, const float* dt_bias, const float* norm_w, float* state, long long slot_floats, long long state_offset, const int* seq_starts, const int* seq_slots, void* y, int y_dtype, long long ldy, float* aux, float* o_raw, int slices, int tokens, int num_seqs, int heads, int kv_heads, int dk, int dv, float unit_eps, float eps);
// conv_shift.cu
int eg_rmsnorm_conv_shift(cudaStream_t stream, const float* residual, const float* gain, float eps, const float* w, float* state, long long slot_floats, const int* token_seq, const int* seq_starts, const int* seq_slots, void* out, void* plain_out, int out_dtype, int tokens, int hidden, int taps, int single);
// conv_shift.cu
int eg_conv_shift(cudaStream_t stream, const float* rows, const float* w, float* state, long long slot_floats, const int* token_seq, const int* seq_starts, const int* seq_slots, void* out, int out_dtype, int tokens, int hidden, int taps, int single);
// conv_shift.cu
int eg_conv_shift_state(cudaStream_t stream, const float* rows, const float* gain, float eps, float* state, long long slot_floats, const int* seq_starts, const int* seq_slots, int num_seqs, int hidden, int taps);
// attention_mixed.cu
int eg_mixed_attention_prepare(cudaStream_t stream, int dtype, const float* proj, long long ld, const float* q_weight, const float* k_weight, float eps, const float* table, int rot_dims, float magnitude, const float* mix, float scale, const int* slot_map, void* k_cache, void* v_cache, long long head_stride, int page_size, long long page_stride, long long pool_slots, void* q_out, int q_dtype, int tokens, int heads, int kv_heads, int dk, int* status);
// attention_mixed.cu
int eg_mixed_attention(cudaStream_t stream, int dtype, const void* q, int q_dtype, const void* k_cache, const void* v_cache, long long head_stride, const int* block_table, int table_stride, const int* token_seq, const int* positions, const float* gate, long long ld_gate, void* out, long long ldo, int num_tokens, int heads, int kv_heads, int dk, int page_size, long long page_stride, int num_pages, int* status);
// attention_mixed_mma.cu
int eg_mixed_attention_mma_takes(int heads, int kv_heads, int dk);
// attention_mixed_mma.cu
int eg_mixed_attention_tiles(cudaStream_t stream, const void* q, const void* k_cache, const void* v_cache, long long head_stride, const int* block_table, int table_stride, const int* positions, const int* tiles, int num_tiles, const float* gate, long long ld_gate, void* out, long long ldo, int heads, int kv_heads, int dk, int page_size, long long page_stride, int num_pages, int* status);
// attention_mixed_mma.cu
int eg_mixed_attention_split(cudaStream_t stream, const void* q, const void* k_cache, const void* v_cache, long long head_stride, const int* block_table, int table_stride, const int* token_seq, const int* positions, const int* token_list, int num_tokens, const float* gate, long long ld_gate, void* out, long long ldo, float* partial_acc, float* partial_ml, int splits, int heads, int kv_heads, int dk, int page_size, long long page_stride, int num_pages, int* status);
// token_side.cu
int eg_add_scaled_rows(cudaStream_t stream, float* residual, const void* delta_a, int dtype_a, const float* scale_a, const void* delta_b, int dtype_b, const float* scale_b, void* rows, int rows_dtype, int tokens, int hidden);
// token_side.cu
int eg_token_side_gate(cudaStream_t stream, int dtype, const float* z, long long ldz, const int* token_ids, const void* table, int vocab, void* g, int tokens, int side, int* status);
// token_side.cu
int eg_add_scaled(cudaStream_t stream, float* residual, const void* delta, int delta_dtype, const float* scale, int tokens, int hidden);
// activation.cu
int eg_squared_relu(cudaStream_t stream, const void* x, int x_dtype, long long ldx, void* out, int out_dtype, long long ldo, int tokens, int n);
// activation.cu
int eg_clamped_glu(cudaStream_t stream, const void* x, int x_dtype, long long ldx, void* out, int out_dtype, long long ldo, int tokens, int n, float limit);
// gemm_skinny.cu
int eg_gemm_skinny_relu2(cudaStream_t stream, int use_pdl, const void* W, long long ldw, int M, int N, int K, const void* x, long long ldx, void* out, long long ldo, int row_blocks, int k_slices, int k_split, float* scratch, int* counters, int* status);
// gemm_skinny.cu
int eg_gemm_skinny_clamped_glu(cudaStream_t stream, int use_pdl, const void* W, long long ldw, int M, int N, int K, const void* x, long long ldx, void* out, long long ldo, int row_blocks, int k_slices, int k_split, float* scratch, int* counters, int* status, float limit);
// gemm_tcgen05.cu
int eg_gemm_tcgen05_pair_relu2(cudaStream_t stream, const void* A, long long lda, const void* W, long long ldw, void* out, long long ldo, int M, int N, int K, int tile_n, int* status);
// gemm_tcgen05.cu
int eg_gemm_tcgen05_pair_glu(cudaStream_t stream, const void* A, long long lda, const void* W, long long ldw, void* out, long long ldo, int M, int N, int K, int* status, float limit);
// gemm_tcgen05.cu
int eg_gemm_tcgen05_grouped_glu(cudaStream_t stream, const void* A, long long lda, const void* W, long long ldw, void* out, long long ldo, int max_rows, int N, int K, int groups, const int* tile_group, int* status, float limit);
// attention_masked.cu
int eg_masked_attention_prepare(cudaStream_t stream, int dtype, const float* proj, long long ld, const float* table, int rot_dims, float magnitude, const int* slot_map, void* k_cache, void* v_cache, int row_stride, long long head_stride, int page_size, long long page_stride, long long pool_slots, void* q_out, int tokens, int heads, int kv_heads, int maps, int dk, int dv, float norm_eps, const float* q_gain, const float* k_gain, int planes, int* status);
// attention_masked.cu
int eg_masked_attention(cudaStream_t stream, int dtype, const void* q, const void* k_cache, const void* v_cache, int row_stride, long long head_stride, const int* block_table, int table_stride, const int* token_seq, const int* positions, const int* token_list, void* out, int out_dtype, long long ldo, int num_tokens, int heads, int kv_heads, int maps, int dk, int dv, int page_size, long long page_stride, int num_pages, int window, int chunk, int keep_first, float scale, float softcap, const float* sinks, float out_scale, int planes, int* status);
// attention_paged.cu
int eg_attention_paged_masked(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache, const int* block_table, int table_stride, const int* token_seq, const int* positions, const int* seq_context, void* out, int out_dtype, int ldo, float* partial_acc, float* partial_ml, int tokens, int num_heads, int num_kv_heads, int maps, int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages, int window, int chunk, int keep_first, float scale, float softcap, const float* sinks, float out_scale, int splits, int* status, int* counters, int use_pdl, const int* token_list);
// attention_paged.cu
int eg_attention_prefill_masked(cudaStream_t stream, const void* q, int ldq, const void* k_cache, const void* v_cache, const int* block_table, int table_stride, const int* positions, const int* tiles, int num_tiles, void* out, int out_dtype, int ldo, int num_heads, int num_kv_heads, int maps, int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages, int window, int chunk, int keep_first, float scale, float softcap, const float* sinks, float out_scale, int* status);
// attention_masked.cu
int eg_attention_map_difference(cudaStream_t stream, const float* maps, void* out, int out_dtype, long long ldo, int tokens, int heads, int dv, float lambda, float eps, float post);
// gated_delta.cu
int eg_gated_delta_channel(cudaStream_t stream, float* qkv, long long ldq, int q_col, int k_col, int v_col, const float* b, long long ldb, int b_col, float* decay, long long ldg, const float* z, long long ldz, const float* a_log, const float* dt_bias, const float* norm_w, float* state, long long slot_floats, long long state_offset, const int* seq_starts, const int* seq_slots, void* y, int y_dtype, long long ldy, float* aux, float* o_raw, int slices, int tokens, int num_seqs, int heads, int kv_heads, int dk, int dv, float unit_eps, float eps, int gate_sigmoid, float out_scale);
// engine_ops.cu
int eg_add_bias_rows(cudaStream_t stream, float* x, long long ld, const float* bias, int rows, int cols);
// engine_ops.cu
int eg_convert_columns(cudaStream_t stream, const float* src, long long lds, void* dst, int dst_dtype, long long ldd, int rows, int cols, int padded);
// activation.cu
int eg_clamped_glu_bias(cudaStream_t stream, const void* x, int x_dtype, long long ldx, const float* bias, void* out, int out_dtype, long long ldo, int tokens, int n, float limit);
// gemm_skinny.cu
int eg_gemm_skinny_clamped_glu_bias(cudaStream_t stream, int use_pdl, const void* W, long long ldw, const float* bias, int M, int N, int K, const void* x, long long ldx, void* out, long long ldo, int row_blocks, int k_slices, int k_split, float* scratch, int* counters, int* status, float limit);
// gemm_tcgen05.cu
int eg_gemm_tcgen05_pair_glu_bias(cudaStream_t stream, const void* A, long long lda, const void* W, long long ldw, const float* bias, void* out, long long ldo, int M, int N, int K, int* status, float limit);
// sandwich.cu
int eg_rmsnorm_add_rows(cudaStream_t stream, float* residual, const void* y, int y_dtype, long long ldy, const float* bias, const float* gain, float eps, void* out, int out_dtype, int tokens, int hidden);
// attention_tcgen05.cu
int eg_attention_prefill_tcgen05_masked(cudaStream_t stream, const void* q, long long ldq, int total_tokens, const void* k_cache, const void* v_cache, const int* block_table, int table_stride, const int* positions, const int* tiles, int num_tiles, void* out, int out_dtype, long long ldo, int num_heads, int num_kv_heads, int maps, int head_dim, int page_size, long long page_stride, long long head_stride, int num_pages, int window, int chunk, int keep_first, float scale, const float* sinks, float out_scale, int* status, int max_parts, int part_tiles, float* partial_o, float* partial_ml, int* queue);
}  // extern "C"
