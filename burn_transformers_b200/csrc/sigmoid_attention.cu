// Attention whose weights are sigmoids of the scores (no softmax, nothing normalised over the keys), with grouped key
// heads, keys and values of different sizes, a sliding window and a run of first positions that stay visible.
//
//   sigmoid_attention_prep  per token: every query and key head is divided by its root mean square (times a weight
//                           shared by the heads), then its first `rot_dims` channels are turned by the token's
//                           position, channel i paired with channel i + rot_dims / 2; every value head is divided by its
//                           root mean square (no weight) and may be mixed with another layer's values of the same token,
//                           v <- (1 - lambda) v + lambda v_other.  All three are rewritten in place (a step of fresh prompts
//                           attends over its own rows); key and value also go into the token's row of the layer's pages,
//                           [key | value] per position and key head.
//   sigmoid_attention       out[t, h] = sum over the visible positions j of sigmoid(q[t, h] . k[j, g] * scale + bias[h])
//                           v[j, g], g = h / (heads / kv_heads); position i sees j <= i with i - j < window or
//                           j < keep_first (window 0: every j <= i).  A block holds a tile of tokens with all query heads
//                           of one key head; for the scores a lane is a key, for the value sum a lane is a set of value
//                           channels.  Sums run over ascending positions in 32-bit, so a row's result does not depend on
//                           what else the step holds.
#include "common.cuh"

namespace bt {

constexpr int SG_WARPS = 8;
constexpr int SG_TK = 32;      // keys per tile: one per lane

template <typename T>
__global__ void __launch_bounds__(128)
sigmoid_attention_prep_kernel(T* __restrict__ proj, long long row_stride, const float* __restrict__ q_weight,
                              const float* __restrict__ k_weight, float eps, const int* __restrict__ positions,
                              const int* __restrict__ token_seq, const float* __restrict__ inv_freq, int rot_dims,
                              const float* __restrict__ mix, const float* __restrict__ v_other,
                              float* __restrict__ v_publish, const int* __restrict__ table, int table_stride,
                              int table_len, int page_size, T* __restrict__ pool, int n_heads, int n_kv_heads, int dim,
                              int vdim) {
  pdl_trigger();
  pdl_wait();
  const long long t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  T* row = proj + t * row_stride;
  const int pos = positions[t], seq = token_seq[t];
  const int lp = pos / page_size;
  const long long page = table[(long long)seq * table_stride + (lp % table_len)];
  const int dkv = dim + vdim, half = rot_dims / 2;
  const float fpos = (float)pos;
  const float lambda = mix != nullptr ? mix[0] : 0.f;
  for (int unit = warp; unit < n_heads + 2 * n_kv_heads; unit += n_warps) {
    if (unit < n_heads + n_kv_heads) {
      // a query or key head: norm with a weight, then the turn
      const bool is_q = unit < n_heads;
      T* src = row + (long long)unit * dim;
      const float* w = is_q ? q_weight : k_weight;
      T* cell = is_q ? nullptr
                     : pool + (((page * n_kv_heads + (unit - n_heads)) * page_size) + (pos - lp * page_size)) * dkv;
      float ss = 0.f;
      for (int c = lane; c < dim; c += 32) {
        const float v = to_float(src[c]);
        ss = fmaf(v, v, ss);
      }
      const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dim + eps);
      for (int i = lane; i < half; i += 32) {
        const float u = to_float(src[i]) * inv * w[i], v = to_float(src[i + half]) * inv * w[i + half];
        float sn, cs;
        sincosf(fpos * inv_freq[i], &sn, &cs);
        const T a = from_float<T>(u * cs - v * sn), b = from_float<T>(v * cs + u * sn);
        src[i] = a;
        src[i + half] = b;
        if (cell != nullptr) { cell[i] = a; cell[i + half] = b; }
      }
      for (int c = 2 * half + lane; c < dim; c += 32) {
        const T a = from_float<T>(to_float(src[c]) * inv * w[c]);
        src[c] = a;
        if (cell != nullptr) cell[c] = a;
      }
    } else {
      const int g = unit - n_heads - n_kv_heads;
      T* src = row + (long long)(n_heads + n_kv_heads) * dim + (long long)g * vdim;
      T* dst = pool + (((page * n_kv_heads + g) * page_size) + (pos - lp * page_size)) * dkv + dim;
      float ss = 0.f;
      for (int c = lane; c < vdim; c += 32) {
        const float v = to_float(src[c]);
        ss = fmaf(v, v, ss);
      }
      const float inv = 1.f / sqrtf(warp_sum(ss) / (float)vdim + eps);
      const long long at = (t * n_kv_heads + g) * vdim;
      for (int c = lane; c < vdim; c += 32) {
        float v = to_float(src[c]) * inv;
        if (v_other != nullptr) v = (1.f - lambda) * v + lambda * v_other[at + c];
        if (v_publish != nullptr) v_publish[at + c] = v;
        dst[c] = from_float<T>(v);
        src[c] = from_float<T>(v);
      }
    }
  }
}

// grid: (token tiles, key heads, sequences).  A row is a (token, query head) pair; a block holds SG_WARPS * RW rows of
// one sequence and key head: `tq` consecutive tokens times the `hb` query heads of the group.  Warp w owns rows w,
// w + SG_WARPS, ...  DVL: value channels per lane (vdim <= 32 * DVL).
template <typename T, int RW, int DVL>
__global__ void __launch_bounds__(SG_WARPS * 32)
sigmoid_attention_kernel(const T* __restrict__ q, long long q_row_stride, const T* __restrict__ pool,
                         const int* __restrict__ table, int table_stride, int table_len, int page_size,
                         const int* __restrict__ seq_start, const int* __restrict__ past_len,
                         const float* __restrict__ bias, T* __restrict__ out, long long out_row_stride, int n_heads,
                         int n_kv_heads, int hb, int tq, int head_tiles, int dim, int vdim, float scale, int window,
                         int keep_first) {
  extern __shared__ float smem[];
  const int ks = dim + 1;                        // key rows one float apart from a multiple of the banks
  float* k_s = smem;                             // [SG_TK][ks]
  float* v_s = k_s + SG_TK * ks;                 // [SG_TK][vdim]
  float* q_s = v_s + SG_TK * vdim;               // [rows][dim]
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.z, g = blockIdx.y / head_tiles, head_tile = blockIdx.y - g * head_tiles;
  const int group_heads = n_heads / n_kv_heads;
  const int first = seq_start[seq], n_new = seq_start[seq + 1] - first, past = past_len[seq];
  const int t0 = blockIdx.x * tq;
  if (t0 >= n_new) return;
  const int h0 = g * group_heads + head_tile * hb, h_end = (g + 1) * group_heads;   // the block's heads: h0 .. h0 + hb - 1
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int ROWS = SG_WARPS * RW;
  const int dkv = dim + vdim;
  for (int i = threadIdx.x; i < ROWS * dim; i += blockDim.x) {
    const int r = i / dim, d = i - r * dim;
    const int tl = r / hb, hl = r - tl * hb;
    const bool ok = r < tq * hb && t0 + tl < n_new && h0 + hl < h_end;
    q_s[i] = ok ? to_float(q[(long long)(first + t0 + tl) * q_row_stride + (long long)(h0 + hl) * dim + d]) : 0.f;
  }
  int row_pos[RW];
  bool row_ok[RW];
  float row_bias[RW], acc[RW][DVL];
#pragma unroll
  for (int i = 0; i < RW; ++i) {
    const int r = warp + i * SG_WARPS;
    const int tl = r / hb, hl = r - tl * hb;
    row_ok[i] = r < tq * hb && t0 + tl < n_new && h0 + hl < h_end;
    row_pos[i] = past + t0 + tl;
    row_bias[i] = row_ok[i] && bias != nullptr ? bias[h0 + hl] : 0.f;
#pragma unroll
    for (int j = 0; j < DVL; ++j) acc[i][j] = 0.f;
  }
  // keys the block may need: the kept first positions, and from the window of its first token to its last token
  const int first_pos = past + t0, last_pos = past + min(t0 + tq, n_new) - 1;
  const int n_tiles = last_pos / SG_TK + 1;
  const int window_tile = window > 0 ? max(0, first_pos - window + 1) / SG_TK : 0;
  const int kept_tiles = window > 0 ? (min(keep_first, last_pos + 1) + SG_TK - 1) / SG_TK : 0;
  for (int tile = 0; tile < n_tiles; ++tile) {
    if (tile >= kept_tiles && tile < window_tile) tile = window_tile;     // (nothing between the two runs is seen)
    const int j0 = tile * SG_TK;
    __syncthreads();  // the previous tile's readers are done (and q_s is complete before the first use)
    for (int i = threadIdx.x; i < SG_TK * dkv; i += blockDim.x) {
      const int kk = i / dkv, d = i - kk * dkv;
      const int j = j0 + kk;
      float v = 0.f;
      if (j <= last_pos) {
        const int lp = j / page_size;
        const long long page = table[(long long)seq * table_stride + (lp % table_len)];
        v = to_float(pool[(((page * n_kv_heads + g) * page_size) + (j - lp * page_size)) * dkv + d]);
      }
      if (d < dim) k_s[kk * ks + d] = v; else v_s[kk * vdim + d - dim] = v;
    }
    __syncthreads();
    float s[RW];
#pragma unroll
    for (int i = 0; i < RW; ++i) s[i] = 0.f;
    const float* krow = k_s + lane * ks;
    for (int d = 0; d < dim; ++d) {
      const float kv = krow[d];
#pragma unroll
      for (int i = 0; i < RW; ++i) s[i] = fmaf(q_s[(warp + i * SG_WARPS) * dim + d], kv, s[i]);
    }
    float p[RW];
#pragma unroll
    for (int i = 0; i < RW; ++i) {
      const int j = j0 + lane, gap = row_pos[i] - j;
      const bool seen = row_ok[i] && gap >= 0 && (window <= 0 || gap < window || j < keep_first);
      p[i] = seen ? 1.f / (1.f + expf(-(s[i] * scale + row_bias[i]))) : 0.f;
    }
    for (int kk = 0; kk < SG_TK; ++kk) {
      float pk[RW];
#pragma unroll
      for (int i = 0; i < RW; ++i) pk[i] = __shfl_sync(0xffffffffu, p[i], kk);
#pragma unroll
      for (int j = 0; j < DVL; ++j) {
        const int c = lane + 32 * j;
        const float v = c < vdim ? v_s[kk * vdim + c] : 0.f;
#pragma unroll
        for (int i = 0; i < RW; ++i) acc[i][j] = fmaf(pk[i], v, acc[i][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < RW; ++i) {
    if (!row_ok[i]) continue;
    const int r = warp + i * SG_WARPS;
    const int tl = r / hb, hl = r - tl * hb;
    const long long token = first + t0 + tl;
#pragma unroll
    for (int j = 0; j < DVL; ++j) {
      const int c = lane + 32 * j;
      if (c < vdim) out[token * out_row_stride + (long long)(h0 + hl) * vdim + c] = from_float<T>(acc[i][j]);
    }
  }
}

// Steps of one token a sequence.  grid: (key heads x head tiles, sequences); a block holds up to SD_ROWS (2, 4 or 8) query
// heads of one key head, and its W warps (up to 16) share the KEYS: warp w takes the visible key tiles w, w + W, ...
// (first those that hold kept first positions and lie before the window, then the window's), each into shared memory
// of its own, so no block barrier stands between tiles.  A tile lies in shared memory as it lies in the page, in the
// cache's element type (16-byte pieces in, 4-byte pieces down; key rows two elements apart from a whole number of
// banks), the queries as 32-bit numbers with a channel's rows side by side (one 16-byte read a channel and four rows).
// For the scores a lane is a key and holds all rows' scores; for the value sum a lane is a set of value channels.  The
// warps' partial sums meet in shared memory and are added in warp order: which warp takes which tile depends on the
// token's position and the window only, so the sum's order does not depend on what else the step holds.
template <typename T> struct SdPiece;
template <> struct SdPiece<float> {            // a 4-byte piece: one number
  static constexpr int N = 1;
  __device__ static void read(const float* p, float (&o)[2]) { o[0] = *p; o[1] = 0.f; }
};
template <> struct SdPiece<__nv_bfloat16> {    // a 4-byte piece: two numbers
  static constexpr int N = 2;
  __device__ static void read(const __nv_bfloat16* p, float (&o)[2]) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    o[0] = f.x; o[1] = f.y;
  }
};

template <typename T, int SD_ROWS, int DVL>
__global__ void __launch_bounds__(512)
sigmoid_attention_decode_kernel(const T* __restrict__ q, long long q_row_stride, const T* __restrict__ pool,
                                const int* __restrict__ table, int table_stride, int table_len, int page_size,
                                const int* __restrict__ seq_start, const int* __restrict__ past_len,
                                const float* __restrict__ bias, T* __restrict__ out, long long out_row_stride,
                                int n_heads, int n_kv_heads, int head_tiles, int dim, int vdim, int ks, float scale,
                                int window, int keep_first) {
  extern __shared__ __align__(16) float smem[];
  constexpr int PN = SdPiece<T>::N;              // numbers in a 4-byte piece
  const int n_warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dkv = dim + vdim;
  float* q_s = smem;                                              // [dim][SD_ROWS]
  const int tile_words = (SG_TK * (ks + vdim) * (int)sizeof(T) + 3) / 4;
  T* k_s = reinterpret_cast<T*>(q_s + SD_ROWS * dim + (size_t)warp * tile_words);   // this warp's [SG_TK][ks]
  T* v_s = k_s + SG_TK * ks;                                      // this warp's [SG_TK][vdim]
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.y, g = blockIdx.x / head_tiles, head_tile = blockIdx.x - g * head_tiles;
  const int group_heads = n_heads / n_kv_heads;
  const int h0 = g * group_heads + head_tile * SD_ROWS;
  const int rows = min(SD_ROWS, (g + 1) * group_heads - h0);
  const long long token = seq_start[seq];
  const int pos = past_len[seq];
  for (int i = threadIdx.x; i < SD_ROWS * dim; i += blockDim.x) {
    const int r = i / dim, d = i - r * dim;
    q_s[d * SD_ROWS + r] = r < rows ? to_float(q[token * q_row_stride + (long long)(h0 + r) * dim + d]) : 0.f;
  }
  __syncthreads();
  float row_bias[SD_ROWS], acc[SD_ROWS][DVL];
#pragma unroll
  for (int r = 0; r < SD_ROWS; ++r) {
    row_bias[r] = r < rows && bias != nullptr ? bias[h0 + r] : 0.f;
#pragma unroll
    for (int j = 0; j < DVL; ++j) acc[r][j] = 0.f;
  }
  const int n_tiles = pos / SG_TK + 1;
  const int window_tile = window > 0 ? max(0, pos - window + 1) / SG_TK : 0;
  const int kept_only = window > 0 ? min((min(keep_first, pos + 1) + SG_TK - 1) / SG_TK, window_tile) : 0;
  const int n_visible = kept_only + n_tiles - window_tile;
  // whole 16-byte pieces that lie in the keys or in the values, never across (else element by element)
  constexpr int V = 16 / (int)sizeof(T);
  const bool pieces_ok = dim % V == 0 && vdim % V == 0 && ks % PN == 0 && (reinterpret_cast<unsigned long long>(pool) & 15) == 0;
  for (int idx = warp; idx < n_visible; idx += n_warps) {
    const int tile = idx < kept_only ? idx : window_tile + (idx - kept_only);
    const int j0 = tile * SG_TK;
    __syncwarp();          // the lanes are done with the tile before
    // a tile of 32 positions never straddles a page (pages hold a multiple of 32 positions), and the rows of one key
    // head lie one after another in a page: the tile is one run of 32 * (dim + vdim) elements.  Positions past the
    // token's own hold whatever an earlier sequence left there (finite numbers): their weights are zero.
    const int lp = j0 / page_size;
    const long long page = table[(long long)seq * table_stride + (lp % table_len)];
    const T* src = pool + (((page * n_kv_heads + g) * page_size) + (j0 - lp * page_size)) * dkv;
    if (pieces_ok) {
      const int per_row = dkv / V, n_pieces = SG_TK * per_row;
#pragma unroll 8
      for (int i = lane; i < n_pieces; i += 32) {
        const int kk = i / per_row, d0 = (i - kk * per_row) * V;
        const uint4 raw = *reinterpret_cast<const uint4*>(src + (long long)i * V);
        uint32_t* dst = reinterpret_cast<uint32_t*>(d0 < dim ? k_s + kk * ks + d0 : v_s + kk * vdim + (d0 - dim));
        dst[0] = raw.x; dst[1] = raw.y; dst[2] = raw.z; dst[3] = raw.w;
      }
    } else {
      for (int i = lane; i < SG_TK * dkv; i += 32) {
        const int kk = i / dkv, d = i - kk * dkv;
        if (d < dim) k_s[kk * ks + d] = src[i]; else v_s[kk * vdim + d - dim] = src[i];
      }
    }
    __syncwarp();
    float s[SD_ROWS];
#pragma unroll
    for (int r = 0; r < SD_ROWS; ++r) s[r] = 0.f;
    const T* krow = k_s + lane * ks;
    int d = 0;
    if (ks % PN == 0) {
#pragma unroll 4
      for (; d + PN <= dim; d += PN) {
        float kv[2];
        SdPiece<T>::read(krow + d, kv);
#pragma unroll
        for (int u = 0; u < PN; ++u) {
          const float* qd = q_s + (d + u) * SD_ROWS;
          if (SD_ROWS % 4 == 0) {
#pragma unroll
            for (int r4 = 0; r4 < SD_ROWS / 4; ++r4) {
              const float4 qv = *reinterpret_cast<const float4*>(qd + 4 * r4);
              s[4 * r4 + 0] = fmaf(qv.x, kv[u], s[4 * r4 + 0]);
              s[4 * r4 + 1] = fmaf(qv.y, kv[u], s[4 * r4 + 1]);
              s[4 * r4 + 2] = fmaf(qv.z, kv[u], s[4 * r4 + 2]);
              s[4 * r4 + 3] = fmaf(qv.w, kv[u], s[4 * r4 + 3]);
            }
          } else {
#pragma unroll
            for (int r = 0; r < SD_ROWS; ++r) s[r] = fmaf(qd[r], kv[u], s[r]);
          }
        }
      }
    }
    for (; d < dim; ++d) {
      const float kv = to_float(krow[d]);
#pragma unroll
      for (int r = 0; r < SD_ROWS; ++r) s[r] = fmaf(q_s[d * SD_ROWS + r], kv, s[r]);
    }
    const int j = j0 + lane, gap = pos - j;
    const bool seen = gap >= 0 && (window <= 0 || gap < window || j < keep_first);
#pragma unroll
    for (int r = 0; r < SD_ROWS; ++r) s[r] = seen ? 1.f / (1.f + expf(-(s[r] * scale + row_bias[r]))) : 0.f;
    const int kk_end = min(SG_TK, pos - j0 + 1);        // (rows past the token's own are never read)
    for (int kk = 0; kk < kk_end; ++kk) {
      float pk[SD_ROWS];
#pragma unroll
      for (int r = 0; r < SD_ROWS; ++r) pk[r] = __shfl_sync(0xffffffffu, s[r], kk);
#pragma unroll
      for (int jj = 0; jj < DVL; ++jj) {
        const int c = lane + 32 * jj;
        const float v = c < vdim ? to_float(v_s[kk * vdim + c]) : 0.f;
#pragma unroll
        for (int r = 0; r < SD_ROWS; ++r) acc[r][jj] = fmaf(pk[r], v, acc[r][jj]);
      }
    }
  }
  // the warps' sums, added in warp order (the tiles' shared memory is free now)
  __syncthreads();
  float* sums = q_s + SD_ROWS * dim;                              // [n_warps][SD_ROWS][vdim]
#pragma unroll
  for (int r = 0; r < SD_ROWS; ++r)
#pragma unroll
    for (int jj = 0; jj < DVL; ++jj) {
      const int c = lane + 32 * jj;
      if (c < vdim) sums[((size_t)warp * SD_ROWS + r) * vdim + c] = acc[r][jj];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < rows * vdim; i += blockDim.x) {
    const int r = i / vdim, c = i - r * vdim;
    float total = 0.f;
    for (int w = 0; w < n_warps; ++w) total += sums[((size_t)w * SD_ROWS + r) * vdim + c];
    out[token * out_row_stride + (long long)(h0 + r) * vdim + c] = from_float<T>(total);
  }
}

template <typename T>
static int launch_sigmoid_attention_decode(const T* q, long long q_row_stride, const T* pool, const int* table,
                                           int table_stride, int table_len, int page_size, const int* seq_start,
                                           const int* past_len, const float* bias, T* out, long long out_row_stride,
                                           int n_seqs, int n_heads, int n_kv_heads, int dim, int vdim, float scale,
                                           int window, int keep_first, cudaStream_t stream) {
  const int group_heads = n_heads / n_kv_heads;
  const int sd_rows = group_heads <= 2 ? 2 : group_heads <= 4 ? 4 : 8;      // rows a lane keeps scores of
  const int head_tiles = (group_heads + sd_rows - 1) / sd_rows;
  const int dvl = (vdim + 31) / 32;
  BT_CHECK(page_size % SG_TK == 0, "sigmoid_attention: pages of %d positions are no whole tiles of %d", page_size, SG_TK);
  // a key row's length in shared memory: a whole number of 4-byte pieces, and an odd number of them, so that the lanes'
  // rows start in different banks
  const int per_word = 4 / (int)sizeof(T);
  int ks = (dim + per_word - 1) / per_word * per_word;
  if ((ks / per_word) % 2 == 0) ks += per_word;
  // as many warps as their tiles fit into shared memory (the warps' sums reuse the tiles' place and are smaller)
  const size_t tile_words = ((size_t)SG_TK * (ks + vdim) * sizeof(T) + 3) / 4;
  auto bytes = [&](int w) {
    const size_t tiles = (size_t)w * tile_words, sums = (size_t)w * sd_rows * vdim;
    return ((size_t)sd_rows * dim + (tiles > sums ? tiles : sums)) * sizeof(float);
  };
  int warps = 16;
  while (warps > 1 && bytes(warps) > 160 * 1024) warps >>= 1;
  const size_t smem = bytes(warps);
  BT_CHECK(smem <= 200 * 1024, "sigmoid_attention: heads of %d + %d channels need %zu bytes of shared memory", dim, vdim,
           smem);
  BT_CHECK(n_seqs <= 65535, "sigmoid_attention: %d sequences are more than a launch takes", n_seqs);
  const dim3 grid(n_kv_heads * head_tiles, n_seqs), block(warps * 32);
#define BT_SD(DVL)                                                                                                     \
  do {                                                                                                                 \
    if (sd_rows == 2) BT_SD_ROWS(2, DVL); else if (sd_rows == 4) BT_SD_ROWS(4, DVL); else BT_SD_ROWS(8, DVL);          \
  } while (0)
#define BT_SD_ROWS(ROWS, DVL)                                                                                          \
  do {                                                                                                                 \
    auto kernel = sigmoid_attention_decode_kernel<T, ROWS, DVL>;                                                       \
    if (smem > 48 * 1024) {                                                                                            \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
      BT_CHECK(e == cudaSuccess, "sigmoid_attention: cannot reserve %zu bytes of shared memory", smem);                \
    }                                                                                                                  \
    BT_PDL_OK("sigmoid_attention_decode",                                                                              \
              launch_pdl(kernel, grid, block, smem, stream, 1, q, q_row_stride, pool, table, table_stride, table_len,  \
                         page_size, seq_start, past_len, bias, out, out_row_stride, n_heads, n_kv_heads, head_tiles,   \
                         dim, vdim, ks, scale, window, keep_first));                                                   \
  } while (0)
  if (dvl <= 1) BT_SD(1);
  else if (dvl <= 2) BT_SD(2);
  else if (dvl <= 4) BT_SD(4);
  else BT_SD(8);
#undef BT_SD
#undef BT_SD_ROWS
  return 0;
}

template <typename T>
static int launch_sigmoid_attention(const T* q, long long q_row_stride, const T* pool, const int* table, int table_stride,
                                    int table_len, int page_size, const int* seq_start, const int* past_len,
                                    const float* bias, T* out, long long out_row_stride, int n_seqs, int max_new,
                                    int n_heads, int n_kv_heads, int dim, int vdim, float scale, int window,
                                    int keep_first, cudaStream_t stream) {
  const int group_heads = n_heads / n_kv_heads;
  const int dvl = (vdim + 31) / 32;
  // rows a block holds: the group's heads times as many tokens as fit (one token in a step of single tokens)
  int rw = dvl <= 2 ? 4 : 2;
  if (max_new == 1 && group_heads <= SG_WARPS) rw = 1;
  else if (max_new == 1 && group_heads <= 2 * SG_WARPS) rw = 2;
  const int rows = SG_WARPS * rw;
  const int hb = group_heads < rows ? group_heads : rows;      // heads of a group a block holds
  const int head_tiles = (group_heads + hb - 1) / hb;
  const int tq = rows / hb;
  const int token_tiles = (max_new + tq - 1) / tq;
  const size_t smem = ((size_t)SG_TK * (dim + 1) + (size_t)SG_TK * vdim + (size_t)rows * dim) * sizeof(float);
  BT_CHECK(smem <= 200 * 1024, "sigmoid_attention: heads of %d + %d channels need %zu bytes of shared memory", dim, vdim,
           smem);
  BT_CHECK(n_kv_heads * head_tiles <= 65535 && n_seqs <= 65535, "sigmoid_attention: bad sizes kv_heads=%d seqs=%d",
           n_kv_heads, n_seqs);
  const dim3 grid(token_tiles, n_kv_heads * head_tiles, n_seqs), block(SG_WARPS * 32);
#define BT_SG(RW, DVL)                                                                                                \
  do {                                                                                                                \
    auto kernel = sigmoid_attention_kernel<T, RW, DVL>;                                                               \
    if (smem > 48 * 1024) {                                                                                           \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
      BT_CHECK(e == cudaSuccess, "sigmoid_attention: cannot reserve %zu bytes of shared memory", smem);               \
    }                                                                                                                 \
    BT_PDL_OK("sigmoid_attention",                                                                                    \
              launch_pdl(kernel, grid, block, smem, stream, 1, q, q_row_stride, pool, table, table_stride, table_len, \
                         page_size, seq_start, past_len, bias, out, out_row_stride, n_heads, n_kv_heads, hb, tq,      \
                         head_tiles, dim, vdim, scale, window, keep_first));                                          \
  } while (0)
#define BT_SG_ROWS(DVL)                                                         \
  do {                                                                          \
    if (rw == 1) BT_SG(1, DVL); else if (rw == 2) BT_SG(2, DVL); else BT_SG(4, DVL); \
  } while (0)
  if (dvl <= 2) BT_SG_ROWS(2);
  else if (dvl <= 4) BT_SG_ROWS(4);
  else BT_SG_ROWS(8);
#undef BT_SG_ROWS
#undef BT_SG
  return 0;
}

}  // namespace bt

extern "C" int bt_sigmoid_attention_prep(void* proj, long long row_stride, const float* q_weight, const float* k_weight,
                                         float eps, const int* positions, const int* token_seq, const float* inv_freq,
                                         int rot_dims, const float* mix, const float* v_other, float* v_publish,
                                         const int* table, int table_stride, int table_len, int page_size, void* pool,
                                         int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim, int dtype,
                                         cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && dim > 0 && vdim > 0 && rot_dims >= 0 && rot_dims % 2 == 0 &&
               rot_dims <= dim,
           "sigmoid_attention_prep: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d rot_dims=%d", n_heads, n_kv_heads, dim,
           vdim, rot_dims);
  if (n_tokens == 0) return 0;
#define BT_SP(T)                                                                                                       \
  BT_PDL_OK("sigmoid_attention_prep",                                                                                  \
            launch_pdl(sigmoid_attention_prep_kernel<T>, dim3(n_tokens), dim3(128), 0, stream, 1, (T*)proj, row_stride, \
                       q_weight, k_weight, eps, positions, token_seq, inv_freq, rot_dims, mix, v_other, v_publish,     \
                       table, table_stride, table_len, page_size, (T*)pool, n_heads, n_kv_heads, dim, vdim))
  if (dtype == kF32) BT_SP(float);
  else if (dtype == kBF16) BT_SP(__nv_bfloat16);
  else return fail("sigmoid_attention_prep: unknown dtype %d", dtype);
#undef BT_SP
  return 0;
}

extern "C" int bt_sigmoid_attention(const void* q, long long q_row_stride, const void* pool, const int* table,
                                    int table_stride, int table_len, int page_size, const int* seq_start,
                                    const int* past_len, const float* bias, void* out, long long out_row_stride,
                                    int n_seqs, int max_new, int n_heads, int n_kv_heads, int dim, int vdim, float scale,
                                    int window, int keep_first, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_seqs >= 0 && max_new >= 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && dim > 0 &&
               vdim > 0 && vdim <= 256 && window >= 0 && keep_first >= 0,
           "sigmoid_attention: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d (up to 256) window=%d keep_first=%d", n_heads,
           n_kv_heads, dim, vdim, window, keep_first);
  if (n_seqs == 0 || max_new == 0) return 0;
  if (max_new == 1 && dtype == kF32)
    return launch_sigmoid_attention_decode((const float*)q, q_row_stride, (const float*)pool, table, table_stride,
                                           table_len, page_size, seq_start, past_len, bias, (float*)out, out_row_stride,
                                           n_seqs, n_heads, n_kv_heads, dim, vdim, scale, window, keep_first, stream);
  if (max_new == 1 && dtype == kBF16)
    return launch_sigmoid_attention_decode((const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)pool, table,
                                           table_stride, table_len, page_size, seq_start, past_len, bias,
                                           (__nv_bfloat16*)out, out_row_stride, n_seqs, n_heads, n_kv_heads, dim, vdim,
                                           scale, window, keep_first, stream);
  if (dtype == kF32)
    return launch_sigmoid_attention((const float*)q, q_row_stride, (const float*)pool, table, table_stride, table_len,
                                    page_size, seq_start, past_len, bias, (float*)out, out_row_stride, n_seqs, max_new,
                                    n_heads, n_kv_heads, dim, vdim, scale, window, keep_first, stream);
  if (dtype == kBF16)
    return launch_sigmoid_attention((const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)pool, table,
                                    table_stride, table_len, page_size, seq_start, past_len, bias, (__nv_bfloat16*)out,
                                    out_row_stride, n_seqs, max_new, n_heads, n_kv_heads, dim, vdim, scale, window,
                                    keep_first, stream);
  return fail("sigmoid_attention: unknown dtype %d", dtype);
}
