// C interface of the kernel library.  Every function returns 0 on success; otherwise
// bt_last_error() holds the reason.  dtype codes: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_runtime.h>

extern "C" {
const char* bt_last_error();
int bt_abi_version();
long long bt_launch_count();

// Fills `out` (128 bytes) with a tensor map of a rows x cols bfloat16 tensor (rows `row_stride` elements apart)
// that is copied in boxes of box_rows x 64 columns with the 128-byte swizzle.
int bt_tensor_map_2d_bf16(void* out, const void* base, unsigned long long rows, unsigned long long cols,
                          unsigned long long row_stride, unsigned box_rows);

int bt_embed(const int* tokens, const int* positions, const void* wte, const void* wpe, float* out, int n_tokens,
             int width, int vocab, int n_positions, float scale, int dtype, int* status, cudaStream_t stream);

int bt_layernorm(const float* x, const int* rows, const float* gamma, const float* beta, void* out, int n_rows,
                 int width, float eps, int out_dtype, cudaStream_t stream);

int bt_linear_simt(const void* A, const void* W, const float* bias, const float* residual, void* out, int M, int N,
                   int K, int w_is_nk, int act, int in_dtype, int out_dtype, cudaStream_t stream);

int bt_kv_append(const void* proj, long long row_stride, int k_offset, int v_offset, const int* positions,
                 const int* token_seq, const int* ctx_len, const int* table, int table_stride, int table_len,
                 int page_size, void* k_pool, void* v_pool, int n_tokens, int n_kv_heads, int head_dim, int dtype,
                 cudaStream_t stream);

int bt_attention_prefill_simt(const void* q, long long q_row_stride, const void* k, const void* v,
                              const int* kv_table, int table_stride, int table_len, int page_size,
                              long long kv_row_stride, void* out, const int* seq_start, const int* past_len,
                              int n_seqs, int max_new, int n_heads, int n_kv_heads, int head_dim, float scale,
                              int causal, int window, int dtype, cudaStream_t stream);

int bt_attention_prefill_tcgen05_supports(int head_dim, int page_size);
// The same kernel for weights sigmoid(score * scale + bias[head]) that are not normalised over the keys.
int bt_sigmoid_attention_tcgen05(const void* q, long long q_rows, long long q_row_stride, const void* k, const void* v,
                                 long long pool_pages, const int* kv_table, int table_stride, int table_len, int page_size,
                                 void* out, int* status, const int* seq_start, const int* past_len, int n_seqs, int max_new,
                                 int n_heads, int n_kv_heads, int head_dim, int v_dim, float scale, const float* bias,
                                 int window, int keep_first, long long pool_row_stride, cudaStream_t stream);
int bt_attention_prefill_tcgen05(const void* q, long long q_rows, long long q_row_stride, const void* k, const void* v,
                                 long long pool_pages, const int* kv_table, int table_stride, int table_len, int page_size,
                                 void* out, int* status, const int* seq_start, const int* past_len, int n_seqs, int max_new,
                                 int n_heads, int n_kv_heads, int head_dim, float scale, int causal, int window,
                                 cudaStream_t stream);

long long bt_attention_decode_scratch_floats(int n_seqs, int n_heads, int head_dim, int n_splits);
// out[M, N] = act(a[M, K] @ w[N, K]^T + bias) (+ residual) for at most 64 bfloat16 rows (made for 17..64).
int bt_linear_mid_supports(int M, int N, int K);
int bt_linear_mid(const void* a, const void* w, const float* bias, const float* residual, void* out, int* status, int M, int N,
                  int K, int act, int out_is_f32, int split, cudaStream_t stream);

// Decode attention on tensor cores (bfloat16, head sizes 16..128 in steps of 16): arguments as bt_attention_decode,
// plus the number of pages of the pools.
int bt_attention_decode_mma_supports(int head_dim);
int bt_attention_decode_mma(const void* q, long long q_row_stride, const void* new_k, const void* new_v, void* k_pool,
                            void* v_pool, long long pool_pages, const int* kv_table, int table_stride, int table_len,
                            void* out, float* scratch, int* tickets, int* status, const int* ctx_len, int n_seqs,
                            int n_heads, int n_kv_heads, int head_dim, float scale, int window, int n_splits, int max_ctx,
                            int merge, cudaStream_t stream);

int bt_attention_decode(const void* q, long long q_row_stride, const void* new_k, const void* new_v, void* k_pool,
                        void* v_pool, const int* kv_table, int table_stride, int table_len, int page_size, void* out,
                        float* scratch, int* tickets, int* status, const int* ctx_len, int n_seqs, int n_heads,
                        int n_kv_heads, int head_dim, float scale, int window, int n_splits, int max_ctx, int merge,
                        int dtype, cudaStream_t stream);

int bt_sample(const float* logits, long long row_stride, int n_rows, int vocab, int do_sample, float temperature,
              int top_k, float top_p, float min_p, const float* uniforms, const unsigned long long* stream_seeds,
              const int* counters, int* out_ids, float* out_logp, cudaStream_t stream);
int bt_advance(const int* ids, int* tokens, int* positions, int* past_len, int* ctx_len, int* counters, int n,
               cudaStream_t stream);
int bt_linear_tcgen05_supports(int M, int N, int K);
int bt_linear_tcgen05(const void* a, const void* w, const float* bias, const float* residual, void* out, int* status,
                      int M, int N, int K, int act, int out_is_f32, cudaStream_t stream);
// out[M, N] = act(x[M, K] @ w[N, K]^T + bias) (+ residual) for at most 128 bfloat16 rows over large weights, on the
// tcgen05 tensor cores with the weights on their M side; split: blocks per cluster along K (0: chosen from the shape).
int bt_linear_few_tcgen05_supports(int M, int N, int K);
int bt_linear_few_tcgen05(const void* x, const void* w, const float* bias, const float* residual, void* out, int* status,
                          int M, int N, int K, int act, int out_is_f32, int split, cudaStream_t stream);
int bt_linear_stream_supports(int M, int N, int K, int fuse_ln);
int bt_linear_stream(const void* a, const float* x32, const int* rows, const float* gamma, const float* beta, float eps,
                     const void* w, const float* bias, const float* residual, void* out, int M, int N, int K, int act,
                     int out_is_f32, int warps_k, cudaStream_t stream);
int bt_linear_skinny_supports(int M, int N, int K, int w_is_nk, int fuse_ln);
int bt_linear_skinny(const void* a, const float* x32, const int* rows, const float* gamma, const float* beta, float eps,
                     const void* w, const float* bias, const float* residual, void* out, int M, int N, int K,
                     int w_is_nk, int act, int out_is_f32, int split, cudaStream_t stream);
// Attention over a latent cache (csrc/latent_attention.cu), the decayed linear recurrence (csrc/lightning.cu) and the
// row-wise kernels between products (csrc/rowwise.cu).
int bt_latent_append(const void* src, long long row_stride, const float* norm_weight, float eps, const int* positions,
                     const int* token_seq, const float* inv_freq, int rot_dims, const int* table, int table_stride,
                     int table_len, int page_size, void* pool, int n_tokens, int rank, int rot, int dtype,
                     cudaStream_t stream);
int bt_latent_gather(const void* pool, const int* positions, const int* token_seq, const int* table, int table_stride,
                     int table_len, int page_size, void* rows, int n_tokens, int dk, int dtype, cudaStream_t stream);
// Causal multi-head attention of fresh prompts on tensor cores with a sink and a gate (csrc/sink_attention_mma.cu).
int bt_sink_attention_supports(int dq, int dv, long long q_row, int q_head, long long k_row, int k_head, long long v_row,
                               int v_head, long long gate_row, int gate_head, long long out_row, int out_head);
int bt_sink_attention(const void* q, long long q_row, int q_head, const void* k, long long k_row, int k_head,
                      const void* v, long long v_row, int v_head, const void* gate, long long gate_row, int gate_head,
                      void* out, long long out_row, int out_head, const int* seq_start, const float* sink, int n_seqs,
                      int max_new, int n_heads, int dq, int dv, float scale, int window, int keep_first, int kv_group,
                      int sigmoid, const float* bias, cudaStream_t stream);
int bt_head_linear(const void* a, long long a_row_stride, int a_head_stride, const void* w, void* out,
                   long long out_row_stride, int out_head_stride, const void* gate, long long gate_row_stride,
                   int gate_head_stride, int n_tokens, int n_heads, int K, int N, int tensor_cores, int dtype,
                   cudaStream_t stream);
long long bt_latent_attention_scratch_floats(int n_tokens, int n_heads, int rank, int n_splits);
int bt_latent_attention(const void* q, long long q_row_stride, const void* pool, const int* table, int table_stride,
                        int table_len, int page_size, const int* seq_start, const int* past_len, const float* sink,
                        void* out, long long out_row_stride, float* part, int n_tokens, int n_seqs, int max_new,
                        int n_heads, int rank, int rot, float scale, int n_splits, int window, int tensor_cores, int merge,
                        int dtype, cudaStream_t stream);
// The steps around the latent attention fused for steps of few tokens (csrc/latent_decode.cu).
int bt_latent_decode_prep(const void* proj, long long row_stride, int q_off, int latent_off, const void* latent_rows,
                          long long latent_row_stride, const void* uk,
                          const float* norm_weight, float eps, const int* positions, const int* token_seq,
                          const float* inv_freq, int rot_dims, const int* table, int table_stride, int table_len,
                          int page_size, void* pool, void* q_latent, int n_tokens, int n_heads, int dim, int rank, int rot,
                          int owns, int dtype, cudaStream_t stream);
int bt_latent_decode_finish(const float* part, const void* mixed_latent, int n_splits, const void* uv, const void* gate,
                            long long gate_row_stride, void* out, long long out_row_stride, int n_tokens, int n_heads,
                            int rank, int vdim, int dtype, cudaStream_t stream);
int bt_latent_attention_rows(int rank, int rot, int dtype, int tensor_cores);
int bt_lightning_scan(const void* proj, long long row_stride, int q_off, int k_off, int v_off, float* state,
                      const int* slots, const int* seq_start, const float* decay, float* out, long long out_row_stride,
                      int n_seqs, int n_heads, int dim, int vdim, int act, int dtype, cudaStream_t stream);
long long bt_lightning_chunked_scratch_floats(int n_seqs, int max_new, int n_heads, int dim, int vdim);
int bt_lightning_chunked(const void* proj, long long row_stride, int q_off, int k_off, int v_off, float* state,
                         const int* slots, const int* seq_start, const float* decay, float* out, long long out_row_stride,
                         float* scratch, int max_new, int n_seqs, int n_heads, int dim, int vdim, int act, int dtype,
                         cudaStream_t stream);
int bt_rmsnorm(const void* x, int x_dtype, long long x_row_stride, const float* weight, const void* gate, int gate_dtype,
               long long gate_row_stride, void* out, int out_dtype, long long out_row_stride, int n_rows, int width,
               int groups, float eps, int gate_rule, cudaStream_t stream);
int bt_rmsnorm_add(const float* x, const float* weight, float* stream_rows, const float* next_weight, void* next_out,
                   int next_dtype, long long n_rows, int width, float eps, float factor, cudaStream_t stream);
// The blend of every row with the row of the token before it, with the kept row per sequence (csrc/rowwise.cu).
int bt_token_shift(const float* x, const float* shift, float* state, const int* slots, const int* seq_start,
                   const int* token_seq, void* out, int out_dtype, long long n_rows, int width, cudaStream_t stream);
// Attention whose weights are sigmoids of the scores (csrc/sigmoid_attention.cu).
int bt_sigmoid_attention_prep(void* proj, long long row_stride, const float* q_weight, const float* k_weight, float eps,
                              const int* positions, const int* token_seq, const float* inv_freq, int rot_dims,
                              const float* mix, const float* v_other, float* v_publish, const int* table,
                              int table_stride, int table_len, int page_size, void* pool, int n_tokens, int n_heads,
                              int n_kv_heads, int dim, int vdim, int dtype, cudaStream_t stream);
int bt_sigmoid_attention(const void* q, long long q_row_stride, const void* pool, const int* table, int table_stride,
                         int table_len, int page_size, const int* seq_start, const int* past_len, const float* bias,
                         void* out, long long out_row_stride, int n_seqs, int max_new, int n_heads, int n_kv_heads,
                         int dim, int vdim, float scale, int window, int keep_first, int dtype, cudaStream_t stream);
int bt_polynorm(const void* x, const float* coef, void* out, long long n_rows, int width, float eps, int dtype,
                cudaStream_t stream);
int bt_rotary_half(const void* src, long long src_row_stride, int src_dtype, float* dst, long long dst_row_stride,
                   const int* positions, const float* inv_freq, int n_tokens, int n_vecs, int len, int dims,
                   int scaled_from, float scale, int tail, cudaStream_t stream);
// A short causal convolution with its state (csrc/short_conv.cu), attention whose heads talk before the softmax
// (csrc/talking_attention.cu) and the selective state-space scan (csrc/selective_scan.cu).
int bt_short_conv(const void* src, long long src_row_stride, int src_dtype, const float* w, const float* bias, float* state,
                  const int* slots, const int* seq_start, const int* token_seq, void* out, long long out_row_stride,
                  int out_dtype, void* raw_out, long long raw_row_stride, int raw_first_group, long long n_tokens,
                  int n_seqs, int channels, int taps, int act, int group, float eps, cudaStream_t stream);
int bt_talking_attention(const void* q, long long q_row_stride, const void* k, const void* v, const int* kv_table,
                         int table_stride, int table_len, int page_size, long long kv_row_stride, const void* gate,
                         long long gate_row_stride, void* out, long long out_row_stride, const int* seq_start,
                         const int* past_len, const float* temp, const float* slope, const float* talk, int n_seqs,
                         int max_new, int n_heads, int n_kv_heads, int head_dim, float scale, float cap, int window,
                         float out_scale, int plain, int n_split, float* parts, int dtype, cudaStream_t stream);
int bt_selective_scan_dt(const void* low, long long low_row_stride, const float* w_dt, const float* b_dt, float* dt,
                         long long n_tokens, int channels, int rank, int dtype, cudaStream_t stream);
int bt_selective_scan(const void* x, long long x_row_stride, const void* z, long long z_row_stride, const float* dt,
                      const void* low, long long low_row_stride, int b_off, int c_off, const float* a_log,
                      const float* d_skip, float* state, const int* slots, const int* seq_start, void* out,
                      long long out_row_stride, int n_seqs, int channels, int n_state, float out_scale, int piece,
                      int max_pieces, float* ends, int dtype, cudaStream_t stream);
int bt_rotary_interleaved(const void* src, long long src_row_stride, int src_vec_stride, void* dst,
                          long long dst_row_stride, int dst_vec_stride, const int* positions, const float* inv_freq,
                          int n_tokens, int n_vecs, int len, int dims, int dtype, cudaStream_t stream);
int bt_gated_activation(const void* x, void* out, long long n_rows, int inner, int act, float limit, int dtype,
                        cudaStream_t stream);
int bt_scale(float* x, long long n, float scale, cudaStream_t stream);
// The matrix memory with exponential gates (csrc/mlstm.cu), routed experts (csrc/moe.cu), and the row-wise kernels they
// added (csrc/rowwise.cu).
int bt_mlstm_scan_fuses(int dim, int vdim);
int bt_mlstm_scan(const void* proj, long long row_stride, int q_off, int k_off, int v_off, int i_off, int f_off,
                  const float* i_bias, const float* f_bias, float cap, float q_scale, float* s, float* n, float* m,
                  const int* slots, const int* seq_start, float* out, long long out_row_stride, const float* norm_w,
                  float eps, int g_off, void* mixed, long long mixed_row_stride, int n_seqs, int n_heads, int dim, int vdim,
                  int dtype, cudaStream_t stream);
long long bt_mlstm_chunked_scratch_floats(long long n_rows, int n_seqs, int max_new, int n_heads, int dim, int vdim);
int bt_mlstm_chunked(const void* proj, long long row_stride, int q_off, int k_off, int v_off, int i_off, int f_off,
                     const float* i_bias, const float* f_bias, float cap, float q_scale, float* s, float* n, float* m,
                     const int* slots, const int* seq_start, float* out, long long out_row_stride, float* scratch,
                     long long n_rows, int max_new, int n_seqs, int n_heads, int dim, int vdim, int dtype,
                     cudaStream_t stream);
int bt_moe_route(const void* x, long long x_row_stride, const void* router, int n_tokens, int K, int E, int top,
                 int n_groups, int keep, float scale, int softmax, const float* choice_bias, int normalise, int* ids,
                 float* weights, int dtype, cudaStream_t stream);
int bt_moe_tile_rows();
int bt_moe_sort(const int* ids, int total, int E, int* offsets, int* tile_first, int* order, int* place,
                cudaStream_t stream);
int bt_moe_expert(int first, const void* a, long long a_row_stride, const void* w, void* out, const int* offsets,
                  const int* tile_first, const int* order, const float* pair_weight, int pairs, int E, int top, int K,
                  int N, int act, float limit, int tensor_cores, int dtype, cudaStream_t stream);
int bt_moe_combine(const float* part, const int* place, float* stream_rows, long long n_tokens, int top, int width,
                   const int* ids, const float* weights, const float* input, int n_stored, int store,
                   cudaStream_t stream);
int bt_add_vector(float* x, const float* vec, long long n_rows, int width, cudaStream_t stream);
int bt_add_rows(float* x, const float* a, const float* b, const float* c, long long n, cudaStream_t stream);

int bt_logit_edits(float* logits, long long row_stride, const int* rows, const int* tokens, const float* vals,
                   int n_edits, int vocab, cudaStream_t stream);
}
