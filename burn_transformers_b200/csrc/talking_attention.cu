// Windowed softmax attention whose heads talk before the softmax, in plain 32-bit arithmetic:
//
//     raw_g(i, j)  = cap * tanh((q_g(i) . k_g(j)) * scale * temp[g] / cap) - slope[g] * (i - j)
//     s_h(i, j)    = sum_g talk[h, g] * raw_g(i, j)
//     o_h(i)       = sum_j softmax_j(s_h(i, .)) v_h(j)          over 0 <= i - j < window (window 0: all j <= i)
//     out_h(i)     = o_h(i) * sigmoid(gate_h(i)) * out_scale
//
// Every head's score of a (query, key) pair is needed before any head's softmax weight is known, so one block owns a
// tile of BQ query tokens of one sequence with ALL heads: warp g computes head g's raw scores against a tile of keys
// (a lane a key), leaves them in shared memory, then warp h mixes them with row h of `talk`, keeps an online softmax
// per query, and accumulates the values (a lane a group of value channels).  Keys and values are read from the step's
// own rows (sequences that start in this step) or from the cache pages (a ring for a window), as KvView says.
// The score plane is never stored.  cap <= 0: no cap; slope or talk null: no bias, no mixing.
#include "common.cuh"

namespace bt {

// talking_attention_mma.cu
int talking_attention_mma(const void* q, long long q_row_stride, const KvView& view, const void* gate,
                          long long gate_row_stride, void* out, long long out_row_stride, const int* seq_start,
                          const int* past_len, const float* temp, const float* slope, const float* talk, int n_seqs,
                          int max_new, int n_heads, int n_kv_heads, int head_dim, float scale, float cap, int window,
                          float out_scale, int n_split, float* parts, cudaStream_t stream, bool* taken);

template <typename T, int BQ, int NV>
__global__ void __launch_bounds__(1024)
talking_attention_kernel(const T* __restrict__ q, long long q_row_stride, KvView kv, const T* __restrict__ gate,
                         long long gate_row_stride, T* __restrict__ out, long long out_row_stride,
                         const int* __restrict__ seq_start, const int* __restrict__ past_len,
                         const float* __restrict__ temp, const float* __restrict__ slope, const float* __restrict__ talk,
                         int n_heads, int n_kv_heads, int head_dim, int bk, float scale, float cap, int window,
                         float out_scale) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.y;
  const int t0 = seq_start[seq], n_new = seq_start[seq + 1] - t0;
  const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x;      // (the last tiles see the most keys: first)
  const int q0 = q_tile * BQ;
  if (q0 >= n_new) return;
  const int nq = min(BQ, n_new - q0);
  const int past = past_len[seq];
  const int kv_len = past + n_new;
  const int H = n_heads, G = n_kv_heads, D = head_dim, DP = head_dim + 1;
  float* Qs = smem;                          // [BQ][H][D], already times scale * temp
  float* Ks = Qs + BQ * H * D;               // [G][bk][DP]
  float* Vs = Ks + G * bk * DP;              // [G][bk][D]
  float* Rs = Vs + G * bk * D;               // [H][BQ][32] raw scores
  float* Ps = Rs + H * BQ * 32;              // [H][BQ][32] softmax weights
  float* Ts = Ps + H * BQ * 32;              // [H][H]
  const int tid = threadIdx.x, lane = tid & 31, head = tid >> 5;
  const int kv_head = head / (H / G);
  for (int i = tid; i < BQ * H * D; i += blockDim.x) {
    const int qi = i / (H * D), rest = i - qi * H * D, h = rest / D;
    Qs[i] = qi < nq ? to_float(q[(long long)(t0 + q0 + qi) * q_row_stride + rest]) * (scale * (temp ? temp[h] : 1.f)) : 0.f;
  }
  for (int i = tid; i < H * H; i += blockDim.x) Ts[i] = talk ? talk[i] : (i / H == i % H ? 1.f : 0.f);
  const float my_slope = slope ? slope[head] : 0.f;
  const int pos_first = past + q0, pos_last = past + q0 + nq - 1;
  const int k_hi = min(kv_len, pos_last + 1);                                  // exclusive
  const int k_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
  const int tile_lo = k_lo / bk, tile_hi = (k_hi + bk - 1) / bk;

  float m[BQ], l[BQ], acc[BQ][NV];
#pragma unroll
  for (int u = 0; u < BQ; ++u) {
    m[u] = -INFINITY;
    l[u] = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[u][i] = 0.f;
  }

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    __syncthreads();
    for (int i = tid; i < G * bk * D; i += blockDim.x) {
      const int g = i / (bk * D), rest = i - g * bk * D, r = rest / D, c = rest - r * D;
      const int kp = tile * bk + r;
      float kx = 0.f, vx = 0.f;
      if (kp >= k_lo && kp < k_hi) {
        kx = to_float(kv_row<T>(kv.k, kv, seq, g, G, D, kp)[c]);
        vx = to_float(kv_row<T>(kv.v, kv, seq, g, G, D, kp)[c]);
      }
      Ks[(g * bk + r) * DP + c] = kx;
      Vs[(g * bk + r) * D + c] = vx;
    }
    __syncthreads();
    const int kp = tile * bk + lane;
    // raw scores of this warp's head
    if (lane < bk) {
      const float* kr = Ks + (kv_head * bk + lane) * DP;
#pragma unroll
      for (int u = 0; u < BQ; ++u) {
        const float* qv = Qs + (u * H + head) * D;
        float s = 0.f;
        for (int c = 0; c < D; ++c) s = fmaf(qv[c], kr[c], s);
        if (cap > 0.f) s = cap * tanhf(s / cap);
        s -= my_slope * (float)(past + q0 + u - kp);
        Rs[(head * BQ + u) * 32 + lane] = s;
      }
    }
    __syncthreads();
    // mixed scores, online softmax, value mix of this warp's head
#pragma unroll
    for (int u = 0; u < BQ; ++u) {
      if (u >= nq) continue;                     // (uniform over the block)
      const int qpos = past + q0 + u;
      bool visible = lane < bk && kp >= k_lo && kp <= qpos;
      if (window > 0) visible = visible && qpos - kp < window;
      float s = 0.f;
      if (lane < bk)
        for (int g = 0; g < H; ++g) s = fmaf(Ts[head * H + g], Rs[(g * BQ + u) * 32 + lane], s);
      s = visible ? s : -INFINITY;
      const float m_new = fmaxf(m[u], warp_max(s));
      if (m_new == -INFINITY) continue;          // (nothing visible in this tile yet: uniform over the warp)
      const float p = visible ? expf(s - m_new) : 0.f;
      const float corr = expf(m[u] - m_new);
      l[u] = l[u] * corr + warp_sum(p);
      m[u] = m_new;
      Ps[(head * BQ + u) * 32 + lane] = p;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[u][i] *= corr;
      const float* pr = Ps + (head * BQ + u) * 32;
      for (int j = 0; j < bk; ++j) {
        const float pj = pr[j];
        const float* vrow = Vs + (kv_head * bk + j) * D;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int c = lane + 32 * i;
          if (c < D) acc[u][i] = fmaf(pj, vrow[c], acc[u][i]);
        }
      }
      __syncwarp();
    }
  }
#pragma unroll
  for (int u = 0; u < BQ; ++u) {
    if (u >= nq) continue;
    const float inv = l[u] > 0.f ? 1.f / l[u] : 0.f;
    const long long t = t0 + q0 + u;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < D) {
        float y = acc[u][i] * inv * out_scale;
        if (gate) y *= 1.f / (1.f + expf(-to_float(gate[t * gate_row_stride + head * D + c])));
        out[t * out_row_stride + head * D + c] = from_float<T>(y);
      }
    }
  }
}

static size_t ta_smem(int bq, int H, int G, int D, int bk) {
  return sizeof(float) * ((size_t)bq * H * D + (size_t)G * bk * (2 * D + 1) + 2 * (size_t)H * bq * 32 + (size_t)H * H);
}

template <typename T, int BQ>
static int launch_talking(const T* q, long long q_row_stride, const KvView& view, const T* gate, long long gate_row_stride,
                          T* out, long long out_row_stride, const int* seq_start, const int* past_len, const float* temp,
                          const float* slope, const float* talk, int n_seqs, int max_new, int n_heads, int n_kv_heads,
                          int head_dim, float scale, float cap, int window, float out_scale, cudaStream_t stream) {
  int bk = 32;
  while (bk > 4 && ta_smem(BQ, n_heads, n_kv_heads, head_dim, bk) > 200 * 1024) bk >>= 1;
  const size_t smem = ta_smem(BQ, n_heads, n_kv_heads, head_dim, bk);
  BT_CHECK(smem <= 200 * 1024, "talking_attention: %d heads over %d key heads of %d channels do not fit shared memory",
           n_heads, n_kv_heads, head_dim);
  const dim3 grid((max_new + BQ - 1) / BQ, n_seqs), block(32 * n_heads);
#define BT_TA(NV)                                                                                                      \
  do {                                                                                                                 \
    auto kern = talking_attention_kernel<T, BQ, NV>;                                                                   \
    if (smem > 48 * 1024)                                                                                              \
      BT_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess,      \
               "talking_attention: cannot reserve %zu bytes of shared memory", smem);                                  \
    BT_PDL_OK("talking_attention", launch_pdl(kern, grid, block, smem, stream, 1, q, q_row_stride, view, gate,         \
                                              gate_row_stride, out, out_row_stride, seq_start, past_len, temp, slope,  \
                                              talk, n_heads, n_kv_heads, head_dim, bk, scale, cap, window, out_scale)); \
  } while (0)
  if (head_dim <= 32) BT_TA(1);
  else if (head_dim <= 64) BT_TA(2);
  else if (head_dim <= 128) BT_TA(4);
  else BT_TA(8);
#undef BT_TA
  return 0;
}

}  // namespace bt

// q, gate, out: the first channel of [tokens, heads * head_dim] views (rows *_row_stride elements apart).  kv_table
// null: keys and values are rows of the step itself (k, v point at their first channel of row 0, rows kv_row_stride
// apart); else pages.  temp, slope [heads] and talk [heads, heads] are 32-bit and may be null.  bfloat16 rows go to the
// tensor-core form (talking_attention_mma.cu) where it takes them, unless `plain` asks for the kernel of this file; there
// a step of at most 16 tokens a sequence may share every sequence's keys among n_split blocks that meet in `parts`.
extern "C" int bt_talking_attention(const void* q, long long q_row_stride, const void* k, const void* v, const int* kv_table,
                                    int table_stride, int table_len, int page_size, long long kv_row_stride,
                                    const void* gate, long long gate_row_stride, void* out, long long out_row_stride,
                                    const int* seq_start, const int* past_len, const float* temp, const float* slope,
                                    const float* talk, int n_seqs, int max_new, int n_heads, int n_kv_heads, int head_dim,
                                    float scale, float cap, int window, float out_scale, int plain, int n_split,
                                    float* parts, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_heads > 0 && n_heads <= 32 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
           "talking_attention: %d query heads (at most 32) over %d key heads", n_heads, n_kv_heads);
  BT_CHECK(head_dim > 0 && head_dim <= 256, "talking_attention: head_dim %d must be 1 .. 256", head_dim);
  BT_CHECK(n_seqs <= 65535 && window >= 0, "talking_attention: too many sequences for one launch, or a negative window");
  if (n_seqs == 0 || max_new == 0) return 0;
  KvView view{k, v, kv_table, table_stride, table_len > 0 ? table_len : 1, page_size > 0 ? page_size : 1, kv_row_stride,
              seq_start};
#define BT_TA_GO(T, BQ)                                                                                              \
  return launch_talking<T, BQ>((const T*)q, q_row_stride, view, (const T*)gate, gate_row_stride, (T*)out,           \
                               out_row_stride, seq_start, past_len, temp, slope, talk, n_seqs, max_new, n_heads,     \
                               n_kv_heads, head_dim, scale, cap, window, out_scale, stream)
  if (dtype == kF32) {
    if (max_new == 1) BT_TA_GO(float, 1);
    BT_TA_GO(float, 4);
  }
  if (dtype == kBF16) {
    if (!plain) {
      bool taken = false;
      const int rc = talking_attention_mma(q, q_row_stride, view, gate, gate_row_stride, out, out_row_stride, seq_start,
                                           past_len, temp, slope, talk, n_seqs, max_new, n_heads, n_kv_heads, head_dim,
                                           scale, cap, window, out_scale, n_split, parts, stream, &taken);
      if (taken || rc) return rc;
    }
    if (max_new == 1) BT_TA_GO(__nv_bfloat16, 1);
    BT_TA_GO(__nv_bfloat16, 4);
  }
#undef BT_TA_GO
  return fail("talking_attention: unknown dtype %d", dtype);
}
