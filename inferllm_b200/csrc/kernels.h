// C prototypes of every kernel entry point of csrc/*.cu, for the C++ core (the kernels themselves
// are documented where they are defined).  Conventions: device pointers, dtype codes 0 = float32 and
// 1 = bfloat16, the last argument is the cudaStream_t; the result is 0, a cudaError_t of the launch or
// ILLM_ERR_BAD_ARG (10001) for sizes the kernel refuses.  Nothing here allocates or synchronises.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// attention_decode.cu
int illm_attention_decode(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, float* part_acc, float* part_ml, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, int n_chunks, void* stream);
int illm_attention_decode_ex(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, float* part_acc, float* part_ml, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, int n_chunks, const float* sinks, const float* gate, int gate_stride, void* stream);
int illm_attention_decode_merge(const float* part_acc, const float* part_ml, const int* token_pos, void* out, int T, int nh, int d, int n_chunks, int chunk_keys, int window, void* stream);
int illm_attention_decode_supported(int d, int g, int page_size);
int illm_attention_decode_static(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, int max_len, char* err_msg, int err_len, void* stream);

// attention_decode_gqa.cu
int illm_attention_decode_gqa(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, float* part_acc, float* part_ml, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, int n_chunks, void* stream);

// attention_decode_ring.cu
int illm_attention_decode_ring(const void* q, int q_stride, const void* kc, const void* vc, long long n_pages, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, float* part_acc, float* part_ml, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, int n_splits, int* err, void* stream);
int illm_attention_decode_ring_ex(const void* q, int q_stride, const void* kc, const void* vc, long long n_pages, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, float* part_acc, float* part_ml, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, int n_splits, int* err, int wide_p, const float* sinks, const float* gate, int gate_stride, void* stream);
int illm_attention_decode_ring_rope(const void* qkv, const float* partials, int splits, long long split_stride, const float* cos_sin, int rot, int table_positions, int write_kv, void* kc, void* vc, long long n_pages, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, float* part_acc, float* part_ml, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, int n_splits, int* err, int* step_err, void* stream);

// attention_generic.cu
int illm_attention_generic(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, void* out, int act_dtype, int T, int nh, int nkv, int d, int page_size, int window, float scale, int dv, const float* sinks, const float* gate, int gate_stride, void* stream);

// attention_mixed.cu
int illm_attention_mixed_supported(int nh, int nkv, int d, int esize);
int illm_attention_mixed(const void* q, int q_stride, const void* kc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, void* out, int act_dtype, int T, int nh, int nkv, int d, int page_size, int window, float scale, const float* r1, const float* r2, const float* mix, const float* gate, int gate_stride, int splits, float* part, void* stream);
int illm_attention_mixed_keys_per_tile(int nh, int nkv, int d, int esize, int has_mix);
// attention_mixed_tc.cu
int illm_attention_mixed_tc_supported(int nh, int nkv, int d);
int illm_attention_mixed_tc(const void* q, int q_stride, const void* kc, const int* block_table, int max_pages, const int* token_pos, const int* cu_q, int B, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale, const float* r1, const float* r2, const float* mix, const float* gate, int gate_stride, int n_sms, void* stream);

// attention_prefill.cu
int illm_attention_prefill(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* cu_q, const int* seq_lens, void* out, int B, int max_q, int nh, int nkv, int d, int page_size, int window, float scale, void* stream);

// attention_prefill_tc.cu
int illm_attention_prefill_tc(const void* q, int q_stride, int T, const void* kc, const void* vc, long long n_pages, const int* block_table, int max_pages, const int* cu_q, const int* seq_lens, void* out, int B, int max_q, int nh, int nkv, int d, int page_size, int window, float scale, int* err, void* stream);

// decay_state.cu
int illm_decay_scan_supported(int d, int dv);
int illm_decay_scan(float* x, int T, int ld, int q_off, int k_off, int v_off, int nh, int d, int dv, int qk_act, int v_act, const float* cos_sin, int rot, int n_pos, float k_scale, const float* decay, float* state, const int* slots, const int* cu_q, const int* token_pos, float* out, int B, int* err, int segments, float* seg_state, void* stream);
int illm_gated_scan(const float* x, int T, int ld, int q_off, int k_off, int v_off, int nh, int qk_div, int d, int dv, const float* ga, const float* gb, float* state, long long state_stride, const int* slots, const int* cu_q, float* out, int B, int segments, float* seg_state, float* seg_gate, void* stream);
int illm_group_norm_gate_ex(const float* o, int T, int width, int group, const float* w, int w_len, float eps, const float* gate, int gate_ld, int gate_act, int gate_first, const float* row_scale, int head, const float* skip_w, const float* skip_x, int skip_ld, void* y, int act_dtype, void* stream);
int illm_group_norm_gate(const float* o, int T, int width, int group, const float* w, int w_len, float eps, const float* gate, int gate_ld, int gate_act, void* y, int act_dtype, void* stream);

int illm_attention_prefill_tc_ex(const void* q, int q_stride, int T, const void* kc, const void* vc, long long n_pages, const int* block_table, int max_pages, const int* cu_q, const int* seq_lens, void* out, int B, int max_q, int nh, int nkv, int d, int page_size, int window, float scale, int* err, int wide_p, const float* sinks, const float* gate, int gate_stride, void* stream);

// bigram_embedding.cu
int illm_bigram_embedding(const int* ids, const int* token_pos, const int* token_seq, const int* cu_q, const int* slots, int* last_token, const void* table, const void* bigram, int table_dtype, float* out, int T, int B, int H, int V, int buckets, long long mul_prev, long long mul_cur, int* err, void* stream);

// delta_state.cu
int illm_delta_rule_supported(int d, int dv, int taps);
int illm_delta_rule(const float* x, int T, int ld, int q_off, int k_off, int v_off, int b_off, const float* a, int nh, int nkv, int d, int dv, int taps, const float* conv_q, const float* conv_k, const float* conv_v, const float* a_log, const float* dt_bias, float q_scale, float* state, long long state_elems, const int* slots, const int* cu_q, const int* token_pos, const int* token_seq, const int* seq_lens, float* qkv, float* g, float* beta, float* out, int B, void* stream);

// gated_state.cu
int illm_mlstm_gates(const float* x, int T, int ld, int q_off, int k_off, int i_off, int f_off, const float* i_bias, const float* f_bias, float cap, float q_scale, int nh, int d, float* state, long long state_stride, long long n_off, long long m_off, const int* slots, const int* cu_q, float* ga, float* gb, float* scale, int B, void* stream);
int illm_ssm_gates(const float* x, int T, int ld, int dt_off, const float* dt_bias, const float* a_log, int nh, float* ga, float* gb, void* stream);

// layernorm.cu
int illm_layernorm_sandwich(float* x, const float* y, const float* wb, const float* w, void* out, int out_dtype, const int* rows, int n_rows, int H, float eps, int write_x, void* stream);

// short_conv.cu
int illm_short_conv(const float* x, int T, int ldx, int x_off, int C, int taps, const float* w, const float* bias, int act, int residual, float* state, long long state_stride, long long state_off, const int* slots, const int* cu_q, const int* token_seq, int B, void* out, int out_dtype, int ldo, int o_off, int update_state, void* stream);

// latent_attention.cu
int illm_latent_prep(const float* x, int ld, int Q, int R, const float* wq, const float* wkv, float eps, const int* token_pos, const int* token_seq, const int* block_table, int max_pages, int page_size, void* cq_out, void* kc, int act_dtype, int T, int* err, void* stream);
int illm_latent_attention_any(const void* q, const void* kc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, void* out, int act_dtype, int T, int H, int R, int page_size, int window, float scale, void* stream);
int illm_head_gemm(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype, int T, int heads, int N, int K, int nn, void* stream);

// moe.cu
int illm_moe_max_tiles(int T, int top, int E, int bm);
int illm_moe_row_tile(int T, int top, int tensor_cores);
int illm_moe_route(const float* logits, const float* bias, int T, int E, int top, int bm, int* expert, float* weight, int* row_of_pair, int* pair_of_row, int* tile_expert, int* tile_row0, int* tile_rows, void* stream);
int illm_moe_route_ex(const float* logits, const float* bias, int T, int E, int top, int bm, int scoring, int groups, int keep, int renorm, int* expert, float* weight, int* row_of_pair, int* pair_of_row, int* tile_expert, int* tile_row0, int* tile_rows, void* stream);
int illm_moe_combine_plus(const float* rows, const int* row_of_pair, const float* weight, const float* plus, float* out, int T, int D, int top, void* stream);
int illm_moe_gemm(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int T, int top, int E, int N, int K, int gated, int act, int bm, int tensor_cores, const int* pair_of_row, const int* tile_expert, const int* tile_row0, const int* tile_rows, void* stream);
int illm_moe_gather_rows(const void* x, void* xs, const int* pair_of_row, int P, int K, int top, void* stream);
int illm_moe_combine(const float* rows, const int* row_of_pair, const float* weight, float* out, int T, int D, int top, void* stream);

// moe_tc.cu
int illm_moe_gemm_tc(const void* xs, const void* w, void* y, int P, int E, int N, int K, int gated, int act, int tiles, const int* tile_expert, const int* tile_row0, const int* tile_rows, int* err, void* stream);

// stream_ops.cu
int illm_gated_act(const void* gu, void* out, int act_dtype, int T, int I, int act, void* stream);
int illm_take_columns(const float* x, int ld, int off, int n_cols, void* y, int act_dtype, int T, void* stream);
int illm_add2_rmsnorm(float* resid, const float* d1, const float* d2, const float* w, void* y, int act_dtype, int T, int H, float eps, void* stream);
int illm_join_rows(const float* a, const float* b, int H, void* y, int act_dtype, int T, void* stream);

// embedding.cu
int illm_embedding(const int* ids, const void* table, int table_dtype, float* out, int T, int H, int V, int* err, void* stream);
int illm_embedding_scaled(const int* ids, const int* token_pos, const void* table, int table_dtype, float* out, int T, int H, int V, float scale, const float* inv_freq, int* err, void* stream);
int illm_set_pdl(int on);
long long illm_launch_count();

// gemm_f32.cu
int illm_gemm_f32_nt(const float* A, const float* W, float* C, int M, int N, int K, int lda, int ldw, int ldc, int* err, void* stream);

// gemm_tc.cu
int illm_gemm_bf16_tc_tune(int stages);
int illm_gemm_bf16_tc(const void* X, const void* W, void* out, int out_dtype, int M, int N, int K, float* ws, int splits, int* err, void* stream, int skip_reduce);
int illm_gemm_bf16_tc_gated(const void* X, const void* W, void* out, int M, int N, int K, int act, int* err, void* stream);
int illm_splitk_reduce(const float* ws, void* out, int out_dtype, long long n, int splits, void* stream);

// gemm_tc2.cu
int illm_gemm_bf16_tc2(const void* X, const void* W, void* out, int out_dtype, int epi, int M, int N, int K, int* err, void* stream);

// postnorm.cu
int illm_scale_add_rmsnorm(float* resid, const void* delta, int delta_dtype, const float* w, void* y, int y_dtype, int n_rows, int H, float alpha, float eps, const float* partials, int splits, long long split_stride, void* stream);

// qk_prep.cu
int illm_qk_prep(const void* x, int x_dtype, int ld, int q_off, int k_off, int v_off, int nh, int nkv, int d, int dv, const float* bq, const float* bk, const float* bv, const float* wq, const float* wk, float eps, const float* cos_sin, int rot, int pairs, int n_pos, const int* token_pos, const int* token_seq, const int* block_table, int max_pages, int page_size, void* q_out, void* kc, void* vc, int act_dtype, int T, int* err, void* stream);

// rmsnorm.cu
int illm_add_rmsnorm(float* resid, const void* delta, const void* w, int w_dtype, void* y, int act_dtype, const int* rows, int n_rows, int H, float eps, int write_resid, void* stream);
int illm_add_rmsnorm_partials(float* resid, const float* partials, int splits, long long split_stride, const void* w, int w_dtype, void* y, int act_dtype, const int* rows, int n_rows, int H, float eps, int write_resid, void* stream);
int illm_residual_add(float* resid, const void* delta, int act_dtype, long long n, void* stream);

// rope_kv.cu
int illm_rope_kv_write(void* qkv, const float* cos_sin, const int* token_pos, const int* token_seq, const int* block_table, int max_pages, void* kc, void* vc, int act_dtype, int T, int nh, int nkv, int d, int rot, int page_size, int write_kv, int table_positions, int* err, void* stream);
int illm_rope_kv_write_partials(void* qkv, const float* partials, int splits, long long split_stride, const float* cos_sin, const int* token_pos, const int* token_seq, const int* block_table, int max_pages, void* kc, void* vc, int act_dtype, int T, int nh, int nkv, int d, int rot, int page_size, int write_kv, int table_positions, int* err, void* stream);

// sampling.cu
int illm_argmax(const float* logits, int B, int V, int ld, int* out, float* scratch_v, int* scratch_i, void* stream);
long long illm_sample_scratch_elems(int B, int V, int top_k, float top_p);
int illm_sample(const float* logits, int B, int V, int ld, float* z_scratch, const int* last_tokens, int n_last, float temp, float penalty, int top_k, float top_p, const float* uniforms, int* out, int* scratch, void* stream);

// swiglu.cu
int illm_swiglu_partials(const float* slices, int P, long long stride, void* out, int T, int I, void* stream);
int illm_swiglu(const void* gu, void* out, int act_dtype, int T, int I, void* stream);

// utility.cu
int illm_fill_random(void* out, int dtype, long long n, unsigned long long key, float std, float mean, void* stream);
int illm_poison_pages(void* k, void* v, long long entry_stride_bytes, int n_entries, long long page_bytes, const int* pages, int n_pages, void* stream);
int illm_selftest_wait_timeout(int* err, long long* result, long long limit_clocks, int code, void* stream);
int illm_convert(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, void* stream);
int illm_gather_i32(const int* src, const int* idx, int* dst, int n, void* stream);
int illm_window_gather(const int* window, int n_last, const int* rows, int* dst, int n, void* stream);
int illm_window_put(int* window, int n_last, const int* rows, int col, const int* toks, int n, void* stream);

// entry points with further parameters (the shorter forms above call them)
int illm_qk_prep_ex(const void* x, int x_dtype, int ld, int q_off, int k_off, int v_off, int nh, int nkv, int d, int dv, const float* bq, const float* bk, const float* bv, const float* wq, const float* wk, float eps, const float* cos_sin, int rot, int pairs, int n_pos, const int* token_pos, const int* token_seq, const int* block_table, int max_pages, int page_size, void* q_out, void* kc, void* vc, int act_dtype, int T, int* err, float qt_coef, int qt_every, void* stream);
int illm_head_gemm_ex(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype, int T, int heads, int N, int K, int nn, int x_ld, int x_hs, int y_ld, int y_hs, void* stream);
int illm_moe_route_ex2(const float* logits, const float* bias, int T, int E, int top, int bm, int scoring, int groups, int keep, int renorm, int group_top, float sum_eps, float weight_scale, int* expert, float* weight, int* row_of_pair, int* pair_of_row, int* tile_expert, int* tile_row0, int* tile_rows, void* stream);
int illm_moe_gemm_ex(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int T, int top, int E, int N, int K, int gated, int act, float act_limit, int bm, int tensor_cores, const int* pair_of_row, const int* tile_expert, const int* tile_row0, const int* tile_rows, void* stream);
int illm_moe_gemm_tc_ex(const void* xs, const void* w, void* y, int P, int E, int N, int K, int gated, int act, float act_limit, int tiles, const int* tile_expert, const int* tile_row0, const int* tile_rows, int* err, void* stream);
// attention_diff.cu
int illm_attention_diff(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, void* out, int act_dtype, int T, int nh, int nkv, int d, int dv, int page_size, int window, float scale, float lambda, float eps, float out_scale, int splits, float* scratch, void* stream);
long long illm_attention_diff_scratch(int T, int nh, int dv, int splits);
int illm_attention_diff_mma_supported(int d, int dv);
int illm_attention_diff_decode_supported(int nh, int nkv, int d, int dv);
int illm_attention_diff_decode(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, void* out, int T, int nh, int nkv, int d, int dv, int page_size, int window, float scale, float lambda, float eps, float out_scale, long long max_len, int splits, float* scratch, void* stream);
int illm_attention_diff_mma(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_pages, const int* cu_q, const int* seq_lens, void* out, int B, int max_q, int nh, int nkv, int d, int dv, int page_size, int window, float scale, float lambda, float eps, float out_scale, void* stream);
// latent_attention.cu
int illm_latent_attention_any_gated(const void* q, const void* kc, const int* block_table, int max_pages, const int* token_pos, const int* token_seq, void* out, int act_dtype, int T, int H, int R, int page_size, int window, float scale, const float* gate, int gate_stride, void* stream);
int illm_latent_rope_prep(const float* x, int ld, int q_off, int H, int d, int dr, int c_off, int R, const float* wkv, float eps, const float* cos_sin, int rot, int pairs, int n_pos, const int* token_pos, const int* token_seq, const int* block_table, int max_pages, int page_size, void* q_nope, int q_f32, void* qa, void* kc, int act_dtype, int T, int* err, void* stream);
// stream_ops.cu
int illm_add_bias(void* y, int dtype, const float* b, int T, int H, void* stream);
int illm_scaled_add_rmsnorm(float* resid, const float* delta, const float* ls, const float* w, void* y, int act_dtype, int T, int H, float eps, void* stream);

#ifdef __cplusplus
}
#endif
