// The small steps around the latent attention, fused for steps of few tokens (decode): with a handful of rows every
// kernel is a link in a chain of launches, so the three steps before the attention and the two after it are one kernel
// each.  One block per (token, head); 32-bit arithmetic; T is the type of projections, weights, cache rows and results.
//
//   latent_decode_prep    q~ = W_uk,h^T q_plain | rotated q_rot  ->  the query as the latent rows meet it;
//                         the block of head 0 also RMS-norms the token's latent, rotates its shared key part and files
//                         both in the page (what bt_latent_append does)
//   latent_decode_finish  joins the attention's splits (or reads its result), multiplies by W_uv,h and by sigmoid(gate)
#include "common.cuh"

namespace bt {

constexpr int LD_THREADS = 256;

// y[j] = sum_k x[k] * W[k][j] for one block: x (K floats) in shared memory, W [K][N] with N contiguous in global memory.
// A thread reads 16 bytes of a row of W at a time; the threads that do not fit beside one another along a row take
// other rows (slices of K), and the slices' partial sums meet in `red` (LD_THREADS * 8 floats of shared memory).
// The results are left in `y` (N <= LD_MAX_N floats of shared memory).  N must be a multiple of the 16-byte piece and W
// 16-byte aligned: `ld_matvec_ok` says so; otherwise the caller loops column by column.
constexpr int LD_MAX_N = 1024;
template <typename T>
__device__ __forceinline__ bool ld_matvec_ok(const T* w, int N) {
  constexpr int VEC = 16 / sizeof(T);
  return N % VEC == 0 && N / VEC <= LD_THREADS && N <= LD_MAX_N && ((unsigned long long)w % 16) == 0;
}

template <typename T>
__device__ __forceinline__ void ld_matvec(const float* x, const T* __restrict__ w, int K, int N, float* red, float* y) {
  constexpr int VEC = 16 / sizeof(T);
  const int groups = N / VEC;                       // threads side by side along a row
  const int slices = LD_THREADS / groups;           // rows of W in flight at once
  const int tid = threadIdx.x, cg = tid % groups, sl = tid / groups;
  float acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
  if (sl < slices) {
#pragma unroll 4
    for (int k = sl; k < K; k += slices) {
      const uint4 raw = *reinterpret_cast<const uint4*>(w + (long long)k * N + cg * VEC);
      const T* e = reinterpret_cast<const T*>(&raw);
      const float xv = x[k];
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[v] = fmaf(xv, to_float(e[v]), acc[v]);
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) red[(sl * groups + cg) * VEC + v] = acc[v];
  }
  __syncthreads();
  for (int j = tid; j < N; j += LD_THREADS) {
    const int g = j / VEC, v = j - g * VEC;
    float sum = 0.f;
    for (int s2 = 0; s2 < slices; ++s2) sum += red[(s2 * groups + g) * VEC + v];
    y[j] = sum;
  }
  __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(LD_THREADS)
latent_decode_prep_kernel(const T* __restrict__ proj, long long row_stride, int q_off,
                          const T* __restrict__ latent_rows, long long latent_row_stride,   // the tokens' [latent | key part]
                          const T* __restrict__ uk,                 // [heads][dim][rank]
                          const float* __restrict__ norm_weight, float eps, const int* __restrict__ positions,
                          const int* __restrict__ token_seq, const float* __restrict__ inv_freq, int rot_dims,
                          const int* __restrict__ table, int table_stride, int table_len, int page_size,
                          T* __restrict__ pool, T* __restrict__ q_latent, int n_heads, int dim, int rank, int rot,
                          int owns) {
  extern __shared__ float sm[];      // [dim] the plain query
  __shared__ float scratch[33];
  __shared__ __align__(16) float red[LD_THREADS * 8];
  __shared__ float y_s[LD_MAX_N];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int pos = positions[t];
  const T* row = proj + (long long)t * row_stride;
  const T* q = row + q_off + (long long)h * (dim + rot);
  for (int d = threadIdx.x; d < dim; d += blockDim.x) sm[d] = to_float(q[d]);
  __syncthreads();
  const int dk = rank + rot;
  T* dst = q_latent + ((long long)t * n_heads + h) * dk;
  const T* w = uk + (long long)h * dim * rank;
  if (ld_matvec_ok(w, rank)) {
    ld_matvec(sm, w, dim, rank, red, y_s);
    for (int r = threadIdx.x; r < rank; r += blockDim.x) dst[r] = from_float<T>(y_s[r]);
  } else {
    for (int r = threadIdx.x; r < rank; r += blockDim.x) {
      float acc = 0.f;
      for (int d = 0; d < dim; ++d) acc = fmaf(sm[d], to_float(w[(long long)d * rank + r]), acc);
      dst[r] = from_float<T>(acc);
    }
  }
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    const float u = to_float(q[dim + 2 * i]), v = to_float(q[dim + 2 * i + 1]);
    dst[rank + 2 * i] = from_float<T>(u * c - v * s);
    dst[rank + 2 * i + 1] = from_float<T>(v * c + u * s);
  }
  for (int c = rot_dims + threadIdx.x; c < rot; c += blockDim.x) dst[rank + c] = q[dim + c];
  if (!owns || h != 0) return;
  // the token's own latent row: norm, rotation, page (the same arithmetic as latent_append_kernel)
  const T* lat = latent_rows + (long long)t * latent_row_stride;
  float ss = 0.f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    const float v = to_float(lat[c]);
    ss += v * v;
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
  const int seq = token_seq[t];
  const int lp = pos / page_size;
  const int page = table[(long long)seq * table_stride + (lp % table_len)];
  T* cell = pool + ((long long)page * page_size + (pos - lp * page_size)) * dk;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) cell[c] = from_float<T>(to_float(lat[c]) * inv * norm_weight[c]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    const float u = to_float(lat[rank + 2 * i]), v = to_float(lat[rank + 2 * i + 1]);
    cell[rank + 2 * i] = from_float<T>(u * c - v * s);
    cell[rank + 2 * i + 1] = from_float<T>(v * c + u * s);
  }
  for (int c = rot_dims + threadIdx.x; c < rot; c += blockDim.x) cell[rank + c] = lat[rank + c];
}

constexpr int LD_MAX_SPLITS = 64;

template <typename T>
__global__ void __launch_bounds__(LD_THREADS)
latent_decode_finish_kernel(const float* __restrict__ part, const T* __restrict__ mixed_latent, int n_splits,
                            const T* __restrict__ uv,               // [heads][rank][vdim]
                            const T* __restrict__ gate, long long gate_row_stride, T* __restrict__ out,
                            long long out_row_stride, int n_heads, int rank, int vdim) {
  extern __shared__ float sm[];      // [rank] the weighted sum of latents, then [LD_MAX_SPLITS] the splits' weights
  float* o_s = sm;
  float* w_s = sm + rank;
  __shared__ __align__(16) float red[LD_THREADS * 8];
  __shared__ float y_s[LD_MAX_N];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const long long unit = (long long)t * n_heads + h;
  if (n_splits > 1) {
    const float* src = part + unit * n_splits * (rank + 2);
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      float m[LD_MAX_SPLITS / 32], l[LD_MAX_SPLITS / 32];
      float top = -INFINITY;
#pragma unroll
      for (int i = 0; i < LD_MAX_SPLITS / 32; ++i) {
        const int s = lane + 32 * i;
        m[i] = s < n_splits ? src[(long long)s * (rank + 2) + rank] : -INFINITY;
        l[i] = s < n_splits ? src[(long long)s * (rank + 2) + rank + 1] : 0.f;
        top = fmaxf(top, m[i]);
      }
      top = warp_max(top);
      float denom = 0.f;
#pragma unroll
      for (int i = 0; i < LD_MAX_SPLITS / 32; ++i) {
        m[i] = m[i] == -INFINITY ? 0.f : expf(m[i] - top);
        denom += l[i] * m[i];
      }
      denom = warp_sum(denom);
      const float inv = denom > 0.f ? 1.f / denom : 0.f;
#pragma unroll
      for (int i = 0; i < LD_MAX_SPLITS / 32; ++i)
        if (lane + 32 * i < n_splits) w_s[lane + 32 * i] = m[i] * inv;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
      float v = 0.f;
#pragma unroll 8
      for (int s = 0; s < n_splits; ++s) v = fmaf(src[(long long)s * (rank + 2) + c], w_s[s], v);
      o_s[c] = v;
    }
  } else {
    const T* src = mixed_latent + unit * rank;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) o_s[c] = to_float(src[c]);
  }
  __syncthreads();
  const T* w = uv + (long long)h * rank * vdim;
  const bool wide = ld_matvec_ok(w, vdim);
  if (wide) ld_matvec(o_s, w, rank, vdim, red, y_s);
  for (int j = threadIdx.x; j < vdim; j += blockDim.x) {
    float acc = wide ? y_s[j] : 0.f;
    if (!wide)
      for (int r = 0; r < rank; ++r) acc = fmaf(o_s[r], to_float(w[(long long)r * vdim + j]), acc);
    if (gate) acc *= 1.f / (1.f + expf(-to_float(gate[(long long)t * gate_row_stride + (long long)h * vdim + j])));
    out[(long long)t * out_row_stride + (long long)h * vdim + j] = from_float<T>(acc);
  }
}

}  // namespace bt

// The queries are the channels from `q_off` on of `proj`'s rows; the tokens' latent rows are `latent_rows` (rows
// `latent_row_stride` elements apart), or, when that is null, the channels from `latent_off` on of the same `proj` rows.
extern "C" int bt_latent_decode_prep(const void* proj, long long row_stride, int q_off, int latent_off,
                                     const void* latent_rows, long long latent_row_stride, const void* uk,
                                     const float* norm_weight, float eps, const int* positions, const int* token_seq,
                                     const float* inv_freq, int rot_dims, const int* table, int table_stride,
                                     int table_len, int page_size, void* pool, void* q_latent, int n_tokens, int n_heads,
                                     int dim, int rank, int rot, int owns, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_heads > 0 && n_heads <= 65535 && dim > 0 && rank > 0 && rot >= 0 && rot_dims >= 0 && rot_dims <= rot &&
           rot_dims % 2 == 0 && dim <= 8192, "latent_decode_prep: bad sizes heads=%d dim=%d rank=%d rot=%d", n_heads, dim, rank, rot);
  if (n_tokens == 0) return 0;
  const dim3 grid(n_tokens, n_heads), block(LD_THREADS);
  const size_t smem = (size_t)dim * sizeof(float);
  const size_t elem = dtype == kF32 ? 4 : 2;
  if (latent_rows == nullptr) {
    latent_rows = (const char*)proj + (size_t)latent_off * elem;
    latent_row_stride = row_stride;
  }
  if (dtype == kF32)
    BT_PDL_OK("latent_decode_prep", launch_pdl(latent_decode_prep_kernel<float>, grid, block, smem, stream, 1,
                                               (const float*)proj, row_stride, q_off, (const float*)latent_rows,
                                               latent_row_stride, (const float*)uk,
                                               norm_weight, eps, positions, token_seq, inv_freq, rot_dims, table,
                                               table_stride, table_len, page_size, (float*)pool, (float*)q_latent, n_heads,
                                               dim, rank, rot, owns));
  else if (dtype == kBF16)
    BT_PDL_OK("latent_decode_prep", launch_pdl(latent_decode_prep_kernel<__nv_bfloat16>, grid, block, smem, stream, 1,
                                               (const __nv_bfloat16*)proj, row_stride, q_off,
                                               (const __nv_bfloat16*)latent_rows, latent_row_stride,
                                               (const __nv_bfloat16*)uk, norm_weight, eps, positions, token_seq, inv_freq,
                                               rot_dims, table, table_stride, table_len, page_size, (__nv_bfloat16*)pool,
                                               (__nv_bfloat16*)q_latent, n_heads, dim, rank, rot, owns));
  else
    return fail("latent_decode_prep: unknown dtype %d", dtype);
  return 0;
}

extern "C" int bt_latent_decode_finish(const float* part, const void* mixed_latent, int n_splits, const void* uv,
                                       const void* gate, long long gate_row_stride, void* out, long long out_row_stride,
                                       int n_tokens, int n_heads, int rank, int vdim, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_heads > 0 && n_heads <= 65535 && rank > 0 && rank <= 8192 && vdim > 0 && n_splits >= 1 &&
           n_splits <= LD_MAX_SPLITS, "latent_decode_finish: bad sizes heads=%d rank=%d vdim=%d splits=%d", n_heads, rank, vdim, n_splits);
  BT_CHECK(n_splits == 1 ? mixed_latent != nullptr : part != nullptr, "latent_decode_finish: the attention's result is missing");
  if (n_tokens == 0) return 0;
  const dim3 grid(n_tokens, n_heads), block(LD_THREADS);
  const size_t smem = (size_t)(rank + LD_MAX_SPLITS) * sizeof(float);
  if (dtype == kF32)
    BT_PDL_OK("latent_decode_finish", launch_pdl(latent_decode_finish_kernel<float>, grid, block, smem, stream, 1, part,
                                                 (const float*)mixed_latent, n_splits, (const float*)uv, (const float*)gate,
                                                 gate_row_stride, (float*)out, out_row_stride, n_heads, rank, vdim));
  else if (dtype == kBF16)
    BT_PDL_OK("latent_decode_finish",
              launch_pdl(latent_decode_finish_kernel<__nv_bfloat16>, grid, block, smem, stream, 1, part,
                         (const __nv_bfloat16*)mixed_latent, n_splits, (const __nv_bfloat16*)uv, (const __nv_bfloat16*)gate,
                         gate_row_stride, (__nv_bfloat16*)out, out_row_stride, n_heads, rank, vdim));
  else
    return fail("latent_decode_finish: unknown dtype %d", dtype);
  return 0;
}
