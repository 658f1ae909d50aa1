// Linear attention with a per-head decay, as a recurrence over a 32-bit state per (sequence, head):
//
//     S_t = decay_h * S_(t-1) + k_t v_t^T        (S: dim x vdim)
//     o_t = S_t^T q_t
//
// q, k, v are act(projection), applied here in 32-bit to the step's projections: act = x * sigmoid(x) (`act` 0) or the
// projection as it is (`act` 1: a caller that has prepared q, k, v itself, for instance rotated them).  Columns of
// S (value channels) never mix, so a block owns a group of value channels of one (sequence, head), keeps its part of
// the state in registers for all tokens of the step, and writes it back once.  Inside a block a value channel belongs
// to SPLIT adjacent lanes, each with DPT of the head's `dim` key channels; their partial outputs meet by shuffles.
// The state lives in `state[slot][head][dim][vdim]`; a sequence that starts finds zeros there.
#include "common.cuh"

namespace bt {

constexpr int LS_TOKENS = 16;  // tokens staged in shared memory at a time

__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float feature(float x, int act) { return act == 0 ? silu(x) : x; }

template <typename T, int DPT, int SPLIT>
__global__ void __launch_bounds__(256)
lightning_scan_kernel(const T* __restrict__ proj, long long row_stride, int q_off, int k_off, int v_off,
                      float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ seq_start,
                      const float* __restrict__ decay, float* __restrict__ out, long long out_row_stride, int n_heads,
                      int dim, int vdim, int cols, int act) {
  extern __shared__ float sm[];
  float* q_s = sm;                          // [LS_TOKENS][dim]
  float* k_s = q_s + LS_TOKENS * dim;       // [LS_TOKENS][dim]
  float* v_s = k_s + LS_TOKENS * dim;       // [LS_TOKENS][cols]
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * cols;
  const int first = seq_start[seq], n_new = seq_start[seq + 1] - first;
  const int part = threadIdx.x % SPLIT, col_local = threadIdx.x / SPLIT;
  const int col = col0 + col_local;
  const bool owns = col_local < cols && col < vdim;
  const int d0 = part * DPT;
  float* s_base = state + (((long long)slots[seq] * n_heads + head) * dim) * vdim;
  float s[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) s[i] = owns && d0 + i < dim ? s_base[(long long)(d0 + i) * vdim + col] : 0.f;
  const float lam = decay[head];
  for (int t0 = 0; t0 < n_new; t0 += LS_TOKENS) {
    const int nt = min(LS_TOKENS, n_new - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * dim; i += blockDim.x) {
      const int t = i / dim, d = i - t * dim;
      const T* row = proj + (long long)(first + t0 + t) * row_stride + (long long)head * dim + d;
      q_s[i] = feature(to_float(row[q_off]), act);
      k_s[i] = feature(to_float(row[k_off]), act);
    }
    for (int i = threadIdx.x; i < nt * cols; i += blockDim.x) {
      const int t = i / cols, c = i - t * cols;
      v_s[i] = col0 + c < vdim
                   ? feature(to_float(proj[(long long)(first + t0 + t) * row_stride + v_off + (long long)head * vdim + col0 + c]), act)
                   : 0.f;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float v = col_local < cols ? v_s[t * cols + col_local] : 0.f;
      const float* kt = k_s + t * dim + d0;
      const float* qt = q_s + t * dim + d0;
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        if (d0 + i < dim) {
          s[i] = fmaf(lam, s[i], kt[i] * v);
          o = fmaf(s[i], qt[i], o);
        }
      }
#pragma unroll
      for (int x = 1; x < SPLIT; x <<= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
      if (owns && part == 0) out[(long long)(first + t0 + t) * out_row_stride + (long long)head * vdim + col] = o;
    }
  }
  if (owns) {
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < dim) s_base[(long long)(d0 + i) * vdim + col] = s[i];
  }
}

template <typename T>
static int launch_lightning(const T* proj, long long row_stride, int q_off, int k_off, int v_off, float* state,
                            const int* slots, const int* seq_start, const float* decay, float* out,
                            long long out_row_stride, int n_seqs, int n_heads, int dim, int vdim, int act, cudaStream_t stream) {
  // DPT key channels per lane, SPLIT lanes per value channel: SPLIT * DPT >= dim
  int dpt, split;
  if (dim <= 32) { dpt = 8; split = 4; }
  else if (dim <= 64) { dpt = 8; split = 8; }
  else if (dim <= 128) { dpt = 16; split = 8; }
  else { dpt = 32; split = 8; }
  BT_CHECK(dim <= 256, "lightning_scan: %d key channels per head; the kernel takes up to 256", dim);
  const int cols = 256 / split < vdim ? 256 / split : vdim;   // value channels per block
  const dim3 grid((vdim + cols - 1) / cols, n_heads, n_seqs), block(256);
  const size_t smem = (size_t)LS_TOKENS * (2 * dim + cols) * sizeof(float);
#define BT_LS(DPT, SPLIT)                                                                                          \
  BT_PDL_OK("lightning_scan", launch_pdl(lightning_scan_kernel<T, DPT, SPLIT>, grid, block, smem, stream, 1, proj, \
                                         row_stride, q_off, k_off, v_off, state, slots, seq_start, decay, out,     \
                                         out_row_stride, n_heads, dim, vdim, cols, act))
  if (dpt == 8 && split == 4) BT_LS(8, 4);
  else if (dpt == 8) BT_LS(8, 8);
  else if (dpt == 16) BT_LS(16, 8);
  else BT_LS(32, 8);
#undef BT_LS
  return 0;
}

}  // namespace bt

extern "C" int bt_lightning_scan(const void* proj, long long row_stride, int q_off, int k_off, int v_off, float* state,
                                 const int* slots, const int* seq_start, const float* decay, float* out,
                                 long long out_row_stride, int n_seqs, int n_heads, int dim, int vdim, int act, int dtype,
                                 cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_heads > 0 && dim > 0 && vdim > 0 && n_seqs >= 0 && n_seqs <= 65535 && n_heads <= 65535,
           "lightning_scan: bad sizes seqs=%d heads=%d dim=%d vdim=%d", n_seqs, n_heads, dim, vdim);
  if (n_seqs == 0) return 0;
  if (dtype == kF32)
    return launch_lightning<float>((const float*)proj, row_stride, q_off, k_off, v_off, state, slots, seq_start, decay,
                                   out, out_row_stride, n_seqs, n_heads, dim, vdim, act, stream);
  if (dtype == kBF16)
    return launch_lightning<__nv_bfloat16>((const __nv_bfloat16*)proj, row_stride, q_off, k_off, v_off, state, slots,
                                           seq_start, decay, out, out_row_stride, n_seqs, n_heads, dim, vdim, act, stream);
  return fail("lightning_scan: unknown dtype %d", dtype);
}

// ---- long runs of new tokens: the same recurrence by chunks ------------------------------------------------------
//
// Unrolled over a chunk of C tokens that starts from the state S_in, the recurrence reads
//
//     o_t   = decay^(t+1) S_in^T q_t + sum_{s <= t} decay^(t-s) (q_t . k_s) v_s          (t, s count inside the chunk)
//     S_out = decay^C S_in + sum_s decay^(C-1-s) k_s v_s^T
//
// so the chunks of a long prompt work side by side: lightning_chunk_kernel forms, per chunk, the sums over s (the part
// of o_t that needs no earlier chunk, and the chunk's own contribution to the state); lightning_prefix_kernel walks the
// chunks of a sequence in order, turning each contribution into the state its chunk starts from; lightning_carry_kernel
// adds decay^(t+1) S_in^T q_t.  Everything is 32-bit multiply-adds; powers of the decay come from powf.
namespace bt {

constexpr int LC = 64;    // tokens per chunk
constexpr int LCP = 68;   // row length of the transposed tiles: 16-byte rows, four-way conflicts at most when they are written

// Tiles of shared memory hold their 64 tokens along the fast axis ([channel][token], rows of LCP floats), so that a
// thread reads four tokens, or four value channels, with one 16-byte load and every product phase is 16 multiply-adds
// per two such loads.  Threads form a 16 x 16 grid; thread (ty, tx) owns a 4 x 4 patch of every product.

// grid (chunks, heads * column blocks, sequences); 256 threads; a block owns 64 value channels.
template <typename T>
__global__ void __launch_bounds__(256)
lightning_chunk_kernel(const T* __restrict__ proj, long long row_stride, int q_off, int k_off, int v_off,
                       const int* __restrict__ seq_start, const float* __restrict__ decay, float* __restrict__ out,
                       long long out_row_stride, float* __restrict__ scratch, int max_chunks, int n_heads, int dim, int vdim,
                       int cols, int col_blocks, int act) {
  extern __shared__ __align__(16) float sm[];
  float* q_t = sm;                       // [dim][LCP]   q_t[d][t]
  float* k_t = q_t + dim * LCP;          // [dim][LCP]   k_t[d][s]
  float* v_s = k_t + dim * LCP;          // [LC][64]     v_s[s][j]
  float* a_t = v_s + LC * 64;            // [LC][LCP]    a_t[s][t] = decay^(t-s) (q_t . k_s), zero for s > t
  float* pw = a_t + LC * LCP;            // [LC + 4] powers of the decay
  pdl_trigger();
  pdl_wait();
  const int chunk = blockIdx.x, seq = blockIdx.z;
  const int head = blockIdx.y / col_blocks, col0 = (blockIdx.y - head * col_blocks) * 64;
  const int first = seq_start[seq], n_new = seq_start[seq + 1] - first;
  if (chunk * LC >= n_new) return;
  const int len = min(LC, n_new - chunk * LC);
  const long long row0 = first + (long long)chunk * LC;
  const float lam = decay[head];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  for (int i = tid; i <= LC; i += 256) pw[i] = powf(lam, (float)i);
  for (int i = tid; i < LC * dim; i += 256) {
    const int t = i / dim, d = i - t * dim;
    float qv = 0.f, kv = 0.f;
    if (t < len) {
      const T* row = proj + (row0 + t) * row_stride + (long long)head * dim + d;
      qv = feature(to_float(row[q_off]), act);
      kv = feature(to_float(row[k_off]), act);
    }
    q_t[d * LCP + t] = qv;
    k_t[d * LCP + t] = kv;
  }
  for (int i = tid; i < LC * 64; i += 256) {
    const int t = i >> 6, c = i & 63;
    v_s[i] = (t < len && col0 + c < vdim)
                 ? feature(to_float(proj[(row0 + t) * row_stride + v_off + (long long)head * vdim + col0 + c]), act) : 0.f;
  }
  __syncthreads();
  // scores of the chunk: tokens t = 4 ty .. and s = 4 tx ..
  {
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    if (tx <= ty) {                      // (patches above the diagonal are zeros)
      for (int d = 0; d < dim; ++d) {
        const float4 qv = *reinterpret_cast<const float4*>(q_t + d * LCP + ty * 4);
        const float4 kv = *reinterpret_cast<const float4*>(k_t + d * LCP + tx * 4);
        const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, ka[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(qa[i], ka[j], acc[i][j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int sx = tx * 4 + j;
      float4 o;
      float* oa = reinterpret_cast<float*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = ty * 4 + i;
        oa[i] = (sx <= t && t < len) ? acc[i][j] * pw[t - sx] : 0.f;
      }
      *reinterpret_cast<float4*>(a_t + sx * LCP + ty * 4) = o;
    }
  }
  __syncthreads();
  // the part of o_t that needs no earlier chunk: tokens 4 ty .., channels 4 tx ..
  {
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const int s_end = min(len, ty * 4 + 4);
    for (int sx = 0; sx < s_end; ++sx) {
      const float4 av = *reinterpret_cast<const float4*>(a_t + sx * LCP + ty * 4);
      const float4 vv = *reinterpret_cast<const float4*>(v_s + sx * 64 + tx * 4);
      const float aa[4] = {av.x, av.y, av.z, av.w}, va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(aa[i], va[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = ty * 4 + i;
      if (t >= len) break;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = col0 + tx * 4 + j;
        if (c < vdim) out[(row0 + t) * out_row_stride + (long long)head * vdim + c] = acc[i][j];
      }
    }
  }
  // the chunk's contribution to the state: sum_s decay^(len-1-s) k_s[i] v_s[c], key channels 4 ty .. (+ 64, ...)
  float* dst = scratch + ((((long long)seq * max_chunks + chunk) * n_heads + head) * dim) * vdim;
  for (int i0 = ty * 4; i0 < dim; i0 += 64) {
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int sx = 0; sx < len; ++sx) {
      const float w = pw[len - 1 - sx];
      const float4 vv = *reinterpret_cast<const float4*>(v_s + sx * 64 + tx * 4);
      const float va[4] = {vv.x * w, vv.y * w, vv.z * w, vv.w * w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float kv = i0 + i < dim ? k_t[(i0 + i) * LCP + sx] : 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(kv, va[j], acc[i][j]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = col0 + tx * 4 + j;
        if (i0 + i < dim && c < vdim) dst[(long long)(i0 + i) * vdim + c] = acc[i][j];
      }
  }
}

// One thread per (sequence, head, state element): walks the sequence's chunks in order; leaves in scratch[chunk] the
// state that chunk STARTS from and in `state` the state after the last one.  Four chunks' contributions are asked for
// at a time, so that the loads do not wait for one another.
__global__ void __launch_bounds__(256)
lightning_prefix_kernel(float* scratch, float* __restrict__ state, const int* __restrict__ slots,
                        const int* __restrict__ seq_start, const float* __restrict__ decay, int max_chunks, int n_heads,
                        int dim, int vdim) {
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int e = blockIdx.x * 256 + threadIdx.x;
  if (e >= dim * vdim) return;
  const int n_new = seq_start[seq + 1] - seq_start[seq];
  const int n_chunks = (n_new + LC - 1) / LC;
  const float lam = decay[head];
  const float full = powf(lam, (float)LC);
  const float tail = powf(lam, (float)(n_new - (n_chunks - 1) * LC));
  float* st = state + (((long long)slots[seq] * n_heads + head) * dim) * vdim + e;
  const long long stride = (long long)n_heads * dim * vdim;
  float* cell = scratch + (((long long)seq * max_chunks) * n_heads + head) * (long long)dim * vdim + e;
  float s = *st;
  for (int c = 0; c < n_chunks; c += 4) {
    float kv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) kv[u] = c + u < n_chunks ? __ldcg(cell + (c + u) * stride) : 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (c + u < n_chunks) {
        cell[(c + u) * stride] = s;
        s = fmaf(c + u == n_chunks - 1 ? tail : full, s, kv[u]);
      }
    }
  }
  *st = s;
}

// out[t] += decay^(t+1) S_in^T q_t for the tokens of a chunk; grid and blocks as lightning_chunk_kernel.
template <typename T>
__global__ void __launch_bounds__(256)
lightning_carry_kernel(const T* __restrict__ proj, long long row_stride, int q_off, const int* __restrict__ seq_start,
                       const float* __restrict__ decay, float* __restrict__ out, long long out_row_stride,
                       const float* __restrict__ scratch, int max_chunks, int n_heads, int dim, int vdim, int cols,
                       int col_blocks, int act) {
  extern __shared__ __align__(16) float sm[];
  float* q_t = sm;                 // [dim][LCP], q_t[d][t] already scaled by decay^(t+1)
  float* s_s = q_t + dim * LCP;    // [dim][64]
  pdl_trigger();
  pdl_wait();
  const int chunk = blockIdx.x, seq = blockIdx.z;
  const int head = blockIdx.y / col_blocks, col0 = (blockIdx.y - head * col_blocks) * 64;
  const int first = seq_start[seq], n_new = seq_start[seq + 1] - first;
  if (chunk * LC >= n_new) return;
  const int len = min(LC, n_new - chunk * LC);
  const long long row0 = first + (long long)chunk * LC;
  const float lam = decay[head];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  for (int i = tid; i < LC * dim; i += 256) {
    const int t = i / dim, d = i - t * dim;
    q_t[d * LCP + t] = t < len ? feature(to_float(proj[(row0 + t) * row_stride + q_off + (long long)head * dim + d]), act) *
                                     powf(lam, (float)(t + 1)) : 0.f;
  }
  const float* src = scratch + ((((long long)seq * max_chunks + chunk) * n_heads + head) * dim) * vdim + col0;
  for (int i = tid; i < dim * 64; i += 256) {
    const int d = i >> 6, c = i & 63;
    s_s[i] = col0 + c < vdim ? src[(long long)d * vdim + c] : 0.f;
  }
  __syncthreads();
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int d = 0; d < dim; ++d) {
    const float4 qv = *reinterpret_cast<const float4*>(q_t + d * LCP + ty * 4);
    const float4 sv = *reinterpret_cast<const float4*>(s_s + d * 64 + tx * 4);
    const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, sa[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(qa[i], sa[j], acc[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = ty * 4 + i;
    if (t >= len) break;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c < vdim) out[(row0 + t) * out_row_stride + (long long)head * vdim + c] += acc[i][j];
    }
  }
}

template <typename T>
static int launch_lightning_chunked(const T* proj, long long row_stride, int q_off, int k_off, int v_off, float* state,
                                    const int* slots, const int* seq_start, const float* decay, float* out,
                                    long long out_row_stride, float* scratch, int max_new, int n_seqs, int n_heads, int dim,
                                    int vdim, int act, cudaStream_t stream) {
  const int cols = 64;
  const int col_blocks = (vdim + cols - 1) / cols;
  const int max_chunks = (max_new + LC - 1) / LC;
  BT_CHECK((long long)n_heads * col_blocks <= 65535, "lightning_scan: %d heads x %d column blocks are too many", n_heads, col_blocks);
  const dim3 grid(max_chunks, n_heads * col_blocks, n_seqs), block(256);
  const size_t smem_a = ((size_t)2 * dim * LCP + (size_t)LC * 64 + (size_t)LC * LCP + LC + 4) * sizeof(float);
  const size_t smem_c = ((size_t)dim * LCP + (size_t)dim * 64) * sizeof(float);
  auto chunk_kernel = lightning_chunk_kernel<T>;
  auto carry_kernel = lightning_carry_kernel<T>;
  if (smem_a > 48 * 1024)
    BT_CHECK(cudaFuncSetAttribute(chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a) == cudaSuccess,
             "lightning_scan: cannot reserve %zu bytes of shared memory", smem_a);
  if (smem_c > 48 * 1024)
    BT_CHECK(cudaFuncSetAttribute(carry_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_c) == cudaSuccess,
             "lightning_scan: cannot reserve %zu bytes of shared memory", smem_c);
  BT_PDL_OK("lightning_chunk", launch_pdl(chunk_kernel, grid, block, smem_a, stream, 1, proj, row_stride, q_off, k_off, v_off,
                                          seq_start, decay, out, out_row_stride, scratch, max_chunks, n_heads, dim, vdim,
                                          cols, col_blocks, act));
  BT_PDL_OK("lightning_prefix", launch_pdl(lightning_prefix_kernel, dim3((dim * vdim + 255) / 256, n_heads, n_seqs), block, 0,
                                           stream, 1, scratch, state, slots, seq_start, decay, max_chunks, n_heads, dim,
                                           vdim));
  BT_PDL_OK("lightning_carry", launch_pdl(carry_kernel, grid, block, smem_c, stream, 1, proj, row_stride, q_off, seq_start,
                                          decay, out, out_row_stride, (const float*)scratch, max_chunks, n_heads, dim, vdim,
                                          cols, col_blocks, act));
  return 0;
}

}  // namespace bt

// Floats of scratch the chunked form needs for runs of up to `max_new` new tokens.
extern "C" long long bt_lightning_chunked_scratch_floats(int n_seqs, int max_new, int n_heads, int dim, int vdim) {
  return (long long)n_seqs * ((max_new + bt::LC - 1) / bt::LC) * n_heads * dim * vdim;
}

// The recurrence for steps that bring long runs of tokens: the same results as bt_lightning_scan (beyond rounding), the
// chunks of a run worked side by side.  `max_new`: no sequence of the step brings more tokens than this.
extern "C" int bt_lightning_chunked(const void* proj, long long row_stride, int q_off, int k_off, int v_off, float* state,
                                    const int* slots, const int* seq_start, const float* decay, float* out,
                                    long long out_row_stride, float* scratch, int max_new, int n_seqs, int n_heads, int dim,
                                    int vdim, int act, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_heads > 0 && dim > 0 && dim <= 256 && vdim > 0 && n_seqs >= 0 && n_seqs <= 65535 && max_new > 0 && scratch,
           "lightning_chunked: bad sizes seqs=%d heads=%d dim=%d vdim=%d max_new=%d", n_seqs, n_heads, dim, vdim, max_new);
  if (n_seqs == 0) return 0;
  if (dtype == kF32)
    return launch_lightning_chunked<float>((const float*)proj, row_stride, q_off, k_off, v_off, state, slots, seq_start,
                                           decay, out, out_row_stride, scratch, max_new, n_seqs, n_heads, dim, vdim, act, stream);
  if (dtype == kBF16)
    return launch_lightning_chunked<__nv_bfloat16>((const __nv_bfloat16*)proj, row_stride, q_off, k_off, v_off, state,
                                                   slots, seq_start, decay, out, out_row_stride, scratch, max_new, n_seqs,
                                                   n_heads, dim, vdim, act, stream);
  return fail("lightning_chunked: unknown dtype %d", dtype);
}
