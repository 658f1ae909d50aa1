// Attention over a latent cache: every head reads the SAME cached row per position.
//
// A layer with a low-rank key/value projection keeps, per position, one row [c | r]: the normalised latent c
// (`rank` channels) and one rotated key part r (`rot` channels) that all heads share.  A head's key is
// [W_uk,h c | r] and its value W_uv,h c.  Because both are linear in c, the up-projections move to the query side:
//
//     score_h(i, j) = scale * ( (W_uk,h^T q_h,plain(i)) . c(j) + q_h,rot(i) . r(j) )
//     mixed_h(i)    = W_uv,h ( sum_j p_h(i, j) c(j) )
//
// so the attention itself is a shared-key attention with key size rank + rot and value = the first `rank` channels
// of the key row: the cache is read once for all heads of a token tile, and nothing per head is ever stored.
//
//   bt_latent_append     RMS-norms the new tokens' latent, rotates their shared key part, files both in the pages
//   bt_head_linear       out[t, h, :] = a[t, h, :] @ W[h]  (per-head products: W_uk^T on queries, W_uv on results),
//                        optionally times sigmoid(gate[t, h, :])
//   bt_latent_attention  scores, softmax with an optional per-head sink in the denominator, value mix; the keys of a
//                        (sequence, row tile) may be cut into splits whose partial results bt_latent_attention_merge joins
//
// Scores, the softmax and every accumulator are 32-bit; T is the type of queries, cache rows and results.
#include "common.cuh"

namespace bt {

// the tensor-core kernel for bfloat16 (latent_attention_mma.cu)
int latent_attention_mma_rows();
bool latent_attention_mma_supports(int rank, int rot);
int launch_latent_attention_mma(const __nv_bfloat16* q, long long q_row_stride, const __nv_bfloat16* pool, const int* table,
                                int table_stride, int table_len, int page_size, const int* seq_start, const int* past_len,
                                const float* sink, __nv_bfloat16* out, long long out_row_stride, float* part, int n_seqs,
                                int max_new, int n_heads, int rank, int rot, float scale, int n_splits, int window,
                                cudaStream_t stream);

// per-head products on tensor cores for bfloat16 (head_linear_mma.cu)
bool head_linear_mma_supports(const void* a, long long a_row_stride, int a_head_stride, const void* w, const void* out,
                              long long out_row_stride, int out_head_stride, const void* gate, long long gate_row_stride,
                              int gate_head_stride, int K, int N);
int launch_head_linear_mma(const __nv_bfloat16* a, long long a_row_stride, int a_head_stride, const __nv_bfloat16* w,
                           __nv_bfloat16* out, long long out_row_stride, int out_head_stride, const __nv_bfloat16* gate,
                           long long gate_row_stride, int gate_head_stride, int n_tokens, int n_heads, int K, int N,
                           cudaStream_t stream);

// ---- filing the latent ------------------------------------------------------------------------------------------

// One block per new token.  src row: [rank latent channels | rot key channels] at `src + t * row_stride`.
// pool[page][page_size][rank + rot]; page of position p: table[seq][(p / page_size) % table_len].
template <typename T>
__global__ void __launch_bounds__(128)
latent_append_kernel(const T* __restrict__ src, long long row_stride, const float* __restrict__ norm_weight, float eps,
                     const int* __restrict__ positions, const int* __restrict__ token_seq,
                     const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ table, int table_stride,
                     int table_len, int page_size, T* __restrict__ pool, int rank, int rot) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = token_seq[t], pos = positions[t];
  const T* row = src + (long long)t * row_stride;
  float ss = 0.f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    const float v = to_float(row[c]);
    ss += v * v;
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
  const int lp = pos / page_size;
  const int page = table[(long long)seq * table_stride + (lp % table_len)];
  T* dst = pool + ((long long)page * page_size + (pos - lp * page_size)) * (rank + rot);
  for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = from_float<T>(to_float(row[c]) * inv * norm_weight[c]);
  // the shared key part: pairs (2i, 2i+1) below rot_dims turn by pos * inv_freq[i]; the rest passes unchanged
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float a = (float)pos * inv_freq[i];
    float s, c;
    sincosf(a, &s, &c);
    const float u = to_float(row[rank + 2 * i]), v = to_float(row[rank + 2 * i + 1]);
    dst[rank + 2 * i] = from_float<T>(u * c - v * s);
    dst[rank + 2 * i + 1] = from_float<T>(v * c + u * s);
  }
  for (int c = rot_dims + threadIdx.x; c < rot; c += blockDim.x) dst[rank + c] = row[rank + c];
}

// rows[t] = the cached row of token t's own position (for steps that want the latents of their tokens side by side)
template <typename T>
__global__ void __launch_bounds__(128)
latent_gather_kernel(const T* __restrict__ pool, const int* __restrict__ positions, const int* __restrict__ token_seq,
                     const int* __restrict__ table, int table_stride, int table_len, int page_size, T* __restrict__ rows,
                     int dk) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = token_seq[t], pos = positions[t];
  const int lp = pos / page_size;
  const int page = table[(long long)seq * table_stride + (lp % table_len)];
  const T* src = pool + ((long long)page * page_size + (pos - lp * page_size)) * dk;
  for (int c = threadIdx.x; c < dk; c += blockDim.x) rows[(long long)t * dk + c] = src[c];
}

// ---- per-head products ------------------------------------------------------------------------------------------

// out[t, h, j] = sum_k a[t, h, k] * W[h][k][j]   (* sigmoid(gate[t, h, j]) if gate)
// a: rows `a_row_stride` apart, head h at a_head_stride * h; out and gate likewise.  A block takes TM tokens of one
// head; a thread owns output columns j, j + blockDim, ... and keeps TM sums per column.
template <typename T, int TM>
__global__ void __launch_bounds__(128)
head_linear_kernel(const T* __restrict__ a, long long a_row_stride, int a_head_stride, const T* __restrict__ w,
                   T* __restrict__ out, long long out_row_stride, int out_head_stride, const T* __restrict__ gate,
                   long long gate_row_stride, int gate_head_stride, int n_tokens, int K, int N) {
  extern __shared__ float a_s[];  // [TM][K]
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y;
  const int t0 = blockIdx.x * TM;
  for (int i = threadIdx.x; i < TM * K; i += blockDim.x) {
    const int m = i / K, k = i - m * K;
    a_s[i] = t0 + m < n_tokens ? to_float(a[(long long)(t0 + m) * a_row_stride + (long long)h * a_head_stride + k]) : 0.f;
  }
  __syncthreads();
  const T* wh = w + (long long)h * K * N;
  for (int j = threadIdx.x; j < N; j += blockDim.x) {
    float acc[TM];
#pragma unroll
    for (int m = 0; m < TM; ++m) acc[m] = 0.f;
    for (int k = 0; k < K; ++k) {
      const float wv = to_float(wh[(long long)k * N + j]);
#pragma unroll
      for (int m = 0; m < TM; ++m) acc[m] = fmaf(a_s[m * K + k], wv, acc[m]);
    }
#pragma unroll
    for (int m = 0; m < TM; ++m) {
      if (t0 + m >= n_tokens) break;
      float v = acc[m];
      if (gate) {
        const float g = to_float(gate[(long long)(t0 + m) * gate_row_stride + (long long)h * gate_head_stride + j]);
        v *= 1.f / (1.f + expf(-g));
      }
      out[(long long)(t0 + m) * out_row_stride + (long long)h * out_head_stride + j] = from_float<T>(v);
    }
  }
}

// ---- the attention ----------------------------------------------------------------------------------------------

constexpr int LA_WARPS = 8;
constexpr int LA_TK = 32;  // keys per tile: one per lane

// grid: (row tiles of a sequence, splits, sequences).  A row is a (token, head) pair; a block holds LA_WARPS * RW rows
// of one sequence, `tq` consecutive tokens times `hb` heads, which all read the same key tiles.  Warp w owns rows
// w, w + LA_WARPS, ...  For the scores a lane is a key; for the value mix a lane is a set of value channels.
// DVL: value channels per lane (rank <= 32 * DVL).
template <typename T, int RW, int DVL>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(const T* __restrict__ q, long long q_row_stride, const T* __restrict__ pool,
                        const int* __restrict__ table, int table_stride, int table_len, int page_size,
                        const int* __restrict__ seq_start, const int* __restrict__ past_len,
                        const float* __restrict__ sink, T* __restrict__ out, long long out_row_stride,
                        float* __restrict__ part, int n_heads, int hb, int tq, int head_tiles, int rank, int rot,
                        float scale, int n_splits, int window) {
  extern __shared__ float smem[];
  const int dk = rank + rot;
  const int ks = dk + 1;                       // key rows one float apart from a multiple of the banks
  float* k_s = smem;                           // [LA_TK][ks]
  float* q_s = smem + LA_TK * ks;              // [rows][dk]
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.z, split = blockIdx.y;
  const int token_tile = blockIdx.x / head_tiles, head_tile = blockIdx.x - token_tile * head_tiles;
  const int first = seq_start[seq], n_new = seq_start[seq + 1] - first, past = past_len[seq];
  const int t0 = token_tile * tq;
  if (t0 >= n_new) return;
  const int h0 = head_tile * hb;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int ROWS = LA_WARPS * RW;
  // row r of the block: token t0 + r / hb, head h0 + r % hb
  for (int i = threadIdx.x; i < ROWS * dk; i += blockDim.x) {
    const int r = i / dk, d = i - r * dk;
    const int tl = r / hb, hl = r - tl * hb;
    const bool ok = r < tq * hb && t0 + tl < n_new && h0 + hl < n_heads;
    q_s[i] = ok ? to_float(q[(long long)(first + t0 + tl) * q_row_stride + (long long)(h0 + hl) * dk + d]) : 0.f;
  }
  int row_pos[RW];
  bool row_ok[RW];
  float m_run[RW], l_run[RW], acc[RW][DVL];
#pragma unroll
  for (int i = 0; i < RW; ++i) {
    const int r = warp + i * LA_WARPS;
    const int tl = r / hb, hl = r - tl * hb;
    row_ok[i] = r < tq * hb && t0 + tl < n_new && h0 + hl < n_heads;
    row_pos[i] = past + t0 + tl;
    // the sink stands in the denominator once: the first split carries it
    const bool has_sink = row_ok[i] && sink != nullptr && split == 0;
    m_run[i] = has_sink ? sink[h0 + hl] : -INFINITY;
    l_run[i] = has_sink ? 1.f : 0.f;
#pragma unroll
    for (int j = 0; j < DVL; ++j) acc[i][j] = 0.f;
  }
  // keys this block may need: from the first one its first token sees (`window` > 0: a row sees the last `window`
  // positions up to its own) to the position of its last token; cut into equal runs of tiles per split
  const int last_pos = past + min(t0 + tq, n_new) - 1;
  const int n_tiles = last_pos / LA_TK + 1;
  const int tile_first = window > 0 ? max(0, past + t0 - window + 1) / LA_TK : 0;
  const int per = (n_tiles - tile_first + n_splits - 1) / n_splits;
  const int tile_lo = tile_first + split * per, tile_hi = min(n_tiles, tile_lo + per);
  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int j0 = tile * LA_TK;
    __syncthreads();  // the previous tile's readers are done (and q_s is complete before the first use)
    for (int i = threadIdx.x; i < LA_TK * dk; i += blockDim.x) {
      const int kk = i / dk, d = i - kk * dk;
      const int j = j0 + kk;
      float v = 0.f;
      if (j <= last_pos) {
        const int lp = j / page_size;
        const int page = table[(long long)seq * table_stride + (lp % table_len)];
        v = to_float(pool[((long long)page * page_size + (j - lp * page_size)) * dk + d]);
      }
      k_s[kk * ks + d] = v;
    }
    __syncthreads();
    // scores: lane = key j0 + lane
    float s[RW];
#pragma unroll
    for (int i = 0; i < RW; ++i) s[i] = 0.f;
    const float* krow = k_s + lane * ks;
    for (int d = 0; d < dk; ++d) {
      const float kv = krow[d];
#pragma unroll
      for (int i = 0; i < RW; ++i) s[i] = fmaf(q_s[(warp + i * LA_WARPS) * dk + d], kv, s[i]);
    }
    float p[RW];
#pragma unroll
    for (int i = 0; i < RW; ++i) {
      const bool seen = row_ok[i] && j0 + lane <= row_pos[i] && (window <= 0 || row_pos[i] - (j0 + lane) < window);
      const float sc = seen ? s[i] * scale : -INFINITY;
      const float m_new = fmaxf(m_run[i], warp_max(sc));
      const float corr = m_new == -INFINITY ? 1.f : expf(m_run[i] - m_new);
      p[i] = seen ? expf(sc - m_new) : 0.f;
      l_run[i] = l_run[i] * corr + warp_sum(p[i]);
      m_run[i] = m_new;
#pragma unroll
      for (int j = 0; j < DVL; ++j) acc[i][j] *= corr;
    }
    // value mix: lane = channels lane, lane + 32, ... of the latent
    for (int kk = 0; kk < LA_TK; ++kk) {
      float pk[RW];
#pragma unroll
      for (int i = 0; i < RW; ++i) pk[i] = __shfl_sync(0xffffffffu, p[i], kk);
#pragma unroll
      for (int j = 0; j < DVL; ++j) {
        const int c = lane + 32 * j;
        const float v = c < rank ? k_s[kk * ks + c] : 0.f;
#pragma unroll
        for (int i = 0; i < RW; ++i) acc[i][j] = fmaf(pk[i], v, acc[i][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < RW; ++i) {
    if (!row_ok[i]) continue;
    const int r = warp + i * LA_WARPS;
    const int tl = r / hb, hl = r - tl * hb;
    const long long token = first + t0 + tl;
    const int head = h0 + hl;
    if (n_splits == 1) {
      const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
#pragma unroll
      for (int j = 0; j < DVL; ++j) {
        const int c = lane + 32 * j;
        if (c < rank) out[token * out_row_stride + (long long)head * rank + c] = from_float<T>(acc[i][j] * inv);
      }
    } else {
      // partial of this split: [token][head][split][rank + 2] = sums, running maximum, denominator
      float* dst = part + ((token * n_heads + head) * n_splits + split) * (rank + 2);
#pragma unroll
      for (int j = 0; j < DVL; ++j) {
        const int c = lane + 32 * j;
        if (c < rank) dst[c] = acc[i][j];
      }
      if (lane == 0) {
        dst[rank] = m_run[i];
        dst[rank + 1] = l_run[i];
      }
    }
  }
}

// Joins the splits' partials.  A warp takes 32 channels of one (token, head): its lanes first turn the splits' maxima
// and denominators into one weight per split (shared memory), then every lane sums its channel over the splits, in
// split order.
constexpr int LA_MAX_SPLITS = 64;

template <typename T>
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* __restrict__ part, T* __restrict__ out, long long out_row_stride, int n_rows,
                              int n_heads, int rank, int n_splits, int groups) {
  __shared__ float weight[4][LA_MAX_SPLITS];
  pdl_trigger();
  pdl_wait();
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + wid;      // (row, group of 32 channels)
  const long long row = unit / groups;
  const int c = (int)(unit - row * groups) * 32 + lane;
  if (row >= n_rows) return;
  const float* src = part + row * n_splits * (rank + 2);
  float m[LA_MAX_SPLITS / 32], l[LA_MAX_SPLITS / 32];
  float top = -INFINITY;
#pragma unroll
  for (int i = 0; i < LA_MAX_SPLITS / 32; ++i) {
    const int s = lane + 32 * i;
    m[i] = s < n_splits ? src[(long long)s * (rank + 2) + rank] : -INFINITY;
    l[i] = s < n_splits ? src[(long long)s * (rank + 2) + rank + 1] : 0.f;
    top = fmaxf(top, m[i]);
  }
  top = warp_max(top);
  float denom = 0.f;
#pragma unroll
  for (int i = 0; i < LA_MAX_SPLITS / 32; ++i) {
    m[i] = m[i] == -INFINITY ? 0.f : expf(m[i] - top);
    denom += l[i] * m[i];
  }
  denom = warp_sum(denom);
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
#pragma unroll
  for (int i = 0; i < LA_MAX_SPLITS / 32; ++i)
    if (lane + 32 * i < n_splits) weight[wid][lane + 32 * i] = m[i] * inv;
  __syncwarp();
  if (c >= rank) return;
  const long long token = row / n_heads;
  const int head = (int)(row - token * n_heads);
  float v = 0.f;
#pragma unroll 8
  for (int s = 0; s < n_splits; ++s) v = fmaf(src[(long long)s * (rank + 2) + c], weight[wid][s], v);
  out[token * out_row_stride + (long long)head * rank + c] = from_float<T>(v);
}

template <typename T>
static int launch_latent_attention(const T* q, long long q_row_stride, const T* pool, const int* table, int table_stride,
                                   int table_len, int page_size, const int* seq_start, const int* past_len,
                                   const float* sink, T* out, long long out_row_stride, float* part, int n_tokens,
                                   int n_seqs, int max_new, int n_heads, int rank, int rot, float scale, int n_splits,
                                   int window, cudaStream_t stream) {
  const int dk = rank + rot;
  const int dvl = (rank + 31) / 32;
  int rw, dvl_t;
  if (dvl <= 2) { rw = 4; dvl_t = 2; }
  else if (dvl <= 4) { rw = 4; dvl_t = 4; }
  else if (dvl <= 8) { rw = 2; dvl_t = 8; }
  else { rw = 2; dvl_t = 16; }
  const int rows = LA_WARPS * rw;
  const int hb = n_heads < rows ? n_heads : rows;
  const int tq = rows / hb;
  const int head_tiles = (n_heads + hb - 1) / hb;
  const int token_tiles = (max_new + tq - 1) / tq;
  const size_t smem = ((size_t)LA_TK * (dk + 1) + (size_t)rows * dk) * sizeof(float);
  BT_CHECK(smem <= 200 * 1024, "latent_attention: rank + rot = %d needs %zu bytes of shared memory", dk, smem);
  const dim3 grid(token_tiles * head_tiles, n_splits, n_seqs), block(LA_WARPS * 32);
#define BT_LA(RW, DVL)                                                                                               \
  do {                                                                                                               \
    auto kernel = latent_attention_kernel<T, RW, DVL>;                                                               \
    if (smem > 48 * 1024) {                                                                                          \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
      BT_CHECK(e == cudaSuccess, "latent_attention: cannot reserve %zu bytes of shared memory", smem);               \
    }                                                                                                                \
    BT_PDL_OK("latent_attention",                                                                                    \
              launch_pdl(kernel, grid, block, smem, stream, 1, q, q_row_stride, pool, table, table_stride, table_len, \
                         page_size, seq_start, past_len, sink, out, out_row_stride, part, n_heads, hb, tq, head_tiles, \
                         rank, rot, scale, n_splits, window));                                                       \
  } while (0)
  if (rw == 4 && dvl_t == 2) BT_LA(4, 2);
  else if (rw == 4 && dvl_t == 4) BT_LA(4, 4);
  else if (dvl_t == 8) BT_LA(2, 8);
  else BT_LA(2, 16);
#undef BT_LA
  return 0;
}

template <typename T>
static int launch_latent_merge(const float* part, T* out, long long out_row_stride, int n_tokens, int n_heads, int rank,
                               int n_splits, cudaStream_t stream) {
  if (n_splits > 1) {
    const int n_rows = n_tokens * n_heads, groups = (rank + 31) / 32;
    const long long units = (long long)n_rows * groups;
    BT_PDL_OK("latent_attention_merge",
              launch_pdl(latent_attention_merge_kernel<T>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, stream, 1,
                         (const float*)part, out, out_row_stride, n_rows, n_heads, rank, n_splits, groups));
  }
  return 0;
}

template <typename T>
static int launch_head_linear(const T* a, long long a_row_stride, int a_head_stride, const T* w, T* out,
                              long long out_row_stride, int out_head_stride, const T* gate, long long gate_row_stride,
                              int gate_head_stride, int n_tokens, int n_heads, int K, int N, cudaStream_t stream) {
  constexpr int TM = 8;
  const size_t smem = (size_t)TM * K * sizeof(float);
  BT_CHECK(smem <= 48 * 1024, "head_linear: K = %d is more than the kernel's rows of shared memory hold", K);
  const dim3 grid((n_tokens + TM - 1) / TM, n_heads), block(128);
  BT_PDL_OK("head_linear", launch_pdl(head_linear_kernel<T, TM>, grid, block, smem, stream, 1, a, a_row_stride,
                                      a_head_stride, w, out, out_row_stride, out_head_stride, gate, gate_row_stride,
                                      gate_head_stride, n_tokens, K, N));
  return 0;
}

}  // namespace bt

extern "C" int bt_latent_append(const void* src, long long row_stride, const float* norm_weight, float eps,
                                const int* positions, const int* token_seq, const float* inv_freq, int rot_dims,
                                const int* table, int table_stride, int table_len, int page_size, void* pool,
                                int n_tokens, int rank, int rot, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(rank > 0 && rot >= 0 && rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0,
           "latent_append: bad sizes rank=%d rot=%d rot_dims=%d", rank, rot, rot_dims);
  BT_CHECK(table_len > 0 && page_size > 0, "latent_append: bad table_len %d or page_size %d", table_len, page_size);
  if (n_tokens == 0) return 0;
  if (dtype == kF32)
    BT_PDL_OK("latent_append", launch_pdl(latent_append_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, 1,
                                          (const float*)src, row_stride, norm_weight, eps, positions, token_seq, inv_freq,
                                          rot_dims, table, table_stride, table_len, page_size, (float*)pool, rank, rot));
  else if (dtype == kBF16)
    BT_PDL_OK("latent_append", launch_pdl(latent_append_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, stream, 1,
                                          (const __nv_bfloat16*)src, row_stride, norm_weight, eps, positions, token_seq,
                                          inv_freq, rot_dims, table, table_stride, table_len, page_size,
                                          (__nv_bfloat16*)pool, rank, rot));
  else
    return fail("latent_append: unknown dtype %d", dtype);
  return 0;
}

extern "C" int bt_latent_gather(const void* pool, const int* positions, const int* token_seq, const int* table,
                                int table_stride, int table_len, int page_size, void* rows, int n_tokens, int dk, int dtype,
                                cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(dk > 0 && table_len > 0 && page_size > 0, "latent_gather: bad sizes dk=%d table_len=%d", dk, table_len);
  if (n_tokens == 0) return 0;
  if (dtype == kF32)
    BT_PDL_OK("latent_gather", launch_pdl(latent_gather_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, 1,
                                          (const float*)pool, positions, token_seq, table, table_stride, table_len,
                                          page_size, (float*)rows, dk));
  else if (dtype == kBF16)
    BT_PDL_OK("latent_gather", launch_pdl(latent_gather_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, stream, 1,
                                          (const __nv_bfloat16*)pool, positions, token_seq, table, table_stride, table_len,
                                          page_size, (__nv_bfloat16*)rows, dk));
  else
    return fail("latent_gather: unknown dtype %d", dtype);
  return 0;
}

extern "C" int bt_head_linear(const void* a, long long a_row_stride, int a_head_stride, const void* w, void* out,
                              long long out_row_stride, int out_head_stride, const void* gate, long long gate_row_stride,
                              int gate_head_stride, int n_tokens, int n_heads, int K, int N, int tensor_cores,
                              int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_heads > 0 && K > 0 && N > 0, "head_linear: bad sizes heads=%d K=%d N=%d", n_heads, K, N);
  if (n_tokens == 0) return 0;
  if (dtype == kBF16 && tensor_cores &&
      head_linear_mma_supports(a, a_row_stride, a_head_stride, w, out, out_row_stride, out_head_stride, gate,
                               gate_row_stride, gate_head_stride, K, N))
    return launch_head_linear_mma((const __nv_bfloat16*)a, a_row_stride, a_head_stride, (const __nv_bfloat16*)w,
                                  (__nv_bfloat16*)out, out_row_stride, out_head_stride, (const __nv_bfloat16*)gate,
                                  gate_row_stride, gate_head_stride, n_tokens, n_heads, K, N, stream);
  if (dtype == kF32)
    return launch_head_linear<float>((const float*)a, a_row_stride, a_head_stride, (const float*)w, (float*)out,
                                     out_row_stride, out_head_stride, (const float*)gate, gate_row_stride,
                                     gate_head_stride, n_tokens, n_heads, K, N, stream);
  if (dtype == kBF16)
    return launch_head_linear<__nv_bfloat16>((const __nv_bfloat16*)a, a_row_stride, a_head_stride,
                                             (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_row_stride,
                                             out_head_stride, (const __nv_bfloat16*)gate, gate_row_stride,
                                             gate_head_stride, n_tokens, n_heads, K, N, stream);
  return fail("head_linear: unknown dtype %d", dtype);
}

// Rows, (token, head) pairs, that one block of the attention kernel holds for this shape and element type.
extern "C" int bt_latent_attention_rows(int rank, int rot, int dtype, int tensor_cores) {
  using namespace bt;
  if (dtype == kBF16 && tensor_cores && latent_attention_mma_supports(rank, rot)) return latent_attention_mma_rows();
  return LA_WARPS * ((rank + 31) / 32 <= 4 ? 4 : 2);
}

extern "C" long long bt_latent_attention_scratch_floats(int n_tokens, int n_heads, int rank, int n_splits) {
  return n_splits > 1 ? (long long)n_tokens * n_heads * n_splits * (rank + 2) : 0;
}

extern "C" int bt_latent_attention(const void* q, long long q_row_stride, const void* pool, const int* table,
                                   int table_stride, int table_len, int page_size, const int* seq_start,
                                   const int* past_len, const float* sink, void* out, long long out_row_stride,
                                   float* part, int n_tokens, int n_seqs, int max_new, int n_heads, int rank, int rot,
                                   float scale, int n_splits, int window, int tensor_cores, int merge, int dtype,
                                   cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_heads > 0 && rank > 0 && rot >= 0 && rank <= 512, "latent_attention: bad sizes heads=%d rank=%d rot=%d (rank "
           "at most 512)", n_heads, rank, rot);
  BT_CHECK(window >= 0, "latent_attention: a window of %d positions", window);
  BT_CHECK(n_splits >= 1 && n_splits <= LA_MAX_SPLITS && (n_splits == 1 || part != nullptr),
           "latent_attention: %d splits need scratch for their partial results", n_splits);
  BT_CHECK(table_len > 0 && page_size > 0 && n_seqs <= 65535, "latent_attention: bad table_len %d, page_size %d or %d "
           "sequences", table_len, page_size, n_seqs);
  if (n_tokens == 0 || n_seqs == 0) return 0;
  if (dtype == kF32) {
    if (int e = launch_latent_attention<float>((const float*)q, q_row_stride, (const float*)pool, table, table_stride,
                                               table_len, page_size, seq_start, past_len, sink, (float*)out,
                                               out_row_stride, part, n_tokens, n_seqs, max_new, n_heads, rank, rot, scale,
                                               n_splits, window, stream))
      return e;
    if (!merge) return 0;
    return launch_latent_merge<float>(part, (float*)out, out_row_stride, n_tokens, n_heads, rank, n_splits, stream);
  }
  if (dtype == kBF16) {
    int e;
    if (tensor_cores && latent_attention_mma_supports(rank, rot))
      e = launch_latent_attention_mma((const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)pool, table,
                                      table_stride, table_len, page_size, seq_start, past_len, sink, (__nv_bfloat16*)out,
                                      out_row_stride, part, n_seqs, max_new, n_heads, rank, rot, scale, n_splits, window,
                                      stream);
    else
      e = launch_latent_attention<__nv_bfloat16>((const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)pool, table,
                                                 table_stride, table_len, page_size, seq_start, past_len, sink,
                                                 (__nv_bfloat16*)out, out_row_stride, part, n_tokens, n_seqs, max_new,
                                                 n_heads, rank, rot, scale, n_splits, window, stream);
    if (e || !merge) return e;
    return launch_latent_merge<__nv_bfloat16>(part, (__nv_bfloat16*)out, out_row_stride, n_tokens, n_heads, rank,
                                              n_splits, stream);
  }
  return fail("latent_attention: unknown dtype %d", dtype);
}
