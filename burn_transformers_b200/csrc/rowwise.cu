// Small row-wise kernels between the products: RMS norm (with an optional sigmoid gate), the interleaved rotation,
// the gated activation of a feed-forward, a scale.  All arithmetic is 32-bit; results are rounded once.
#include "common.cuh"

namespace bt {

// what a gate's pre-activation g multiplies a row by: sigmoid(g) (rule 0) or g * sigmoid(g) (rule 1)
__device__ __forceinline__ float gate_value(float g, int rule) {
  const float s = 1.f / (1.f + expf(-g));
  return rule == 1 ? g * s : s;
}

// out[r, c] = x[r, c] / sqrt(mean_c(x[r]^2) + eps) * weight[c]  (* sigmoid(gate[r, c]) if gate)
// With `groups` > 1 a row is `groups` runs of `width` channels, each normed by its own root mean square (heads side by
// side); weight and gate go on over all channels of the row.
template <typename TIn, typename TGate, typename TOut>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const TIn* __restrict__ x, long long x_row_stride, const float* __restrict__ weight,
               const TGate* __restrict__ gate, long long gate_row_stride, TOut* __restrict__ out,
               long long out_row_stride, int width, int groups, float eps, int gate_rule) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x / groups, first = (blockIdx.x - r * groups) * width;
  const TIn* src = x + (long long)r * x_row_stride + first;
  weight += first;
  if (gate) gate += first;
  out += first;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = to_float(src[c]);
    ss += v * v;
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = to_float(src[c]) * inv * weight[c];
    if (gate) v *= gate_value(to_float(gate[(long long)r * gate_row_stride + c]), gate_rule);
    out[(long long)r * out_row_stride + c] = from_float<TOut>(v);
  }
}

// The same with a warp per run of at most 32 * NV channels: the run stays in registers, read once, no block barrier.
template <typename TIn, typename TGate, typename TOut, int NV>
__global__ void __launch_bounds__(128)
rmsnorm_warp_kernel(const TIn* __restrict__ x, long long x_row_stride, const float* __restrict__ weight,
                    const TGate* __restrict__ gate, long long gate_row_stride, TOut* __restrict__ out,
                    long long out_row_stride, int width, int groups, long long items, float eps, int gate_rule) {
  pdl_trigger();
  pdl_wait();
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= items) return;
  const int lane = threadIdx.x & 31;
  const long long r = item / groups;
  const int first = (int)(item - r * groups) * width;
  const TIn* src = x + r * x_row_stride + first;
  float v[NV], ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    v[i] = c < width ? to_float(src[c]) : 0.f;
    ss = fmaf(v[i], v[i], ss);
  }
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)width + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < width) {
      float y = v[i] * inv * weight[first + c];
      if (gate) y *= gate_value(to_float(gate[r * gate_row_stride + first + c]), gate_rule);
      out[r * out_row_stride + first + c] = from_float<TOut>(y);
    }
  }
}

// dst[t, v, :] = src[t, v, :] with the pairs (2i, 2i+1), i < dims/2, turned by positions[t] * inv_freq[i]; the
// channels from `dims` to `len` are copied.  src and dst may be the same memory.
template <typename T>
__global__ void __launch_bounds__(128)
rotary_interleaved_kernel(const T* src, long long src_row_stride, int src_vec_stride, T* dst, long long dst_row_stride,
                          int dst_vec_stride, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                          int n_vecs, int len, int dims) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  const int half = dims / 2, units = half + (len - dims);   // a unit: one pair, or one copied channel
  for (int i = threadIdx.x; i < n_vecs * units; i += blockDim.x) {
    const int v = i / units, u = i - v * units;
    const T* s = src + (long long)t * src_row_stride + (long long)v * src_vec_stride;
    T* d = dst + (long long)t * dst_row_stride + (long long)v * dst_vec_stride;
    if (u < half) {
      float sn, cs;
      sincosf(pos * inv_freq[u], &sn, &cs);
      const float a = to_float(s[2 * u]), b = to_float(s[2 * u + 1]);
      d[2 * u] = from_float<T>(a * cs - b * sn);
      d[2 * u + 1] = from_float<T>(b * cs + a * sn);
    } else {
      d[dims + (u - half)] = s[dims + (u - half)];
    }
  }
}

// out[r, j] = act(x[r, j]) * x[r, inner + j]  (or the clamped pair rule of common.cuh: gated_pair)
template <typename T>
__global__ void __launch_bounds__(256)
gated_activation_kernel(const T* __restrict__ x, T* __restrict__ out, long long n_rows, int inner, int act,
                        float limit) {
  pdl_trigger();
  pdl_wait();
  const long long total = n_rows * inner;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / inner;
    const int j = (int)(i - r * inner);
    const float g = to_float(x[r * 2 * inner + j]), u = to_float(x[r * 2 * inner + inner + j]);
    out[i] = from_float<T>(gated_pair(g, u, act, limit));
  }
}

// The same for bfloat16 rows whose halves are whole 16-byte pieces: a thread takes 8 channels at a time.
__global__ void __launch_bounds__(256)
gated_activation_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, long long n_rows,
                               int inner, int act, float limit) {
  pdl_trigger();
  pdl_wait();
  const int pieces = inner / 8;
  const long long total = n_rows * pieces;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / pieces;
    const int j = (int)(i - r * pieces) * 8;
    const uint4 gv = *reinterpret_cast<const uint4*>(x + r * 2 * inner + j);
    const uint4 uv = *reinterpret_cast<const uint4*>(x + r * 2 * inner + inner + j);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
      o2[e] = __floats2bfloat162_rn(gated_pair(g.x, u.x, act, limit), gated_pair(g.y, u.y, act, limit));
    }
    *reinterpret_cast<uint4*>(out + r * inner + j) = ov;
  }
}

__global__ void __launch_bounds__(256) scale_kernel(float* __restrict__ x, long long n, float scale) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] *= scale;
}

// x[r, c] += vec[c]: one learned vector added to every row of the 32-bit stream
__global__ void __launch_bounds__(256)
add_vector_kernel(float* __restrict__ x, const float* __restrict__ vec, long long n_rows, int width) {
  pdl_trigger();
  pdl_wait();
  const long long total = n_rows * width;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    x[i] += vec[i % width];
}

// x += a (+ b) (+ c), element by element, in this order: what branches of a layer that ran side by side left in buffers
// of their own joins the 32-bit stream
__global__ void __launch_bounds__(256)
add_rows_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ c,
                long long n) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = x[i] + a[i];
    if (b) v += b[i];
    if (c) v += c[i];
    x[i] = v;
  }
}

template <typename TIn, typename TGate>
static int launch_rmsnorm(const TIn* x, long long xs, const float* w, const TGate* gate, long long gs, void* out,
                          long long os, int n_rows, int width, int groups, float eps, int out_dtype, int gate_rule,
                          cudaStream_t stream) {
  width /= groups;
  const long long items = (long long)n_rows * groups;
  if (width <= 1024) {
    const dim3 wgrid((unsigned)((items + 3) / 4));
#define BT_RW(TOUT, NV)                                                                                              \
  BT_PDL_OK("rmsnorm", launch_pdl(rmsnorm_warp_kernel<TIn, TGate, TOUT, NV>, wgrid, dim3(128), 0, stream, 1, x, xs, w, \
                                  gate, gs, (TOUT*)out, os, width, groups, items, eps, gate_rule))
    if (out_dtype == kF32) {
      if (width <= 128) BT_RW(float, 4); else BT_RW(float, 32);
    } else {
      if (width <= 128) BT_RW(__nv_bfloat16, 4); else BT_RW(__nv_bfloat16, 32);
    }
#undef BT_RW
    return 0;
  }
  const int threads = 256;
  const dim3 grid((unsigned)n_rows * groups);
  if (out_dtype == kF32)
    BT_PDL_OK("rmsnorm", launch_pdl(rmsnorm_kernel<TIn, TGate, float>, grid, dim3(threads), 0, stream, 1, x, xs, w,
                                    gate, gs, (float*)out, os, width, groups, eps, gate_rule));
  else
    BT_PDL_OK("rmsnorm", launch_pdl(rmsnorm_kernel<TIn, TGate, __nv_bfloat16>, grid, dim3(threads), 0, stream, 1, x,
                                    xs, w, gate, gs, (__nv_bfloat16*)out, os, width, groups, eps, gate_rule));
  return 0;
}

}  // namespace bt

extern "C" int bt_rmsnorm(const void* x, int x_dtype, long long x_row_stride, const float* weight, const void* gate,
                          int gate_dtype, long long gate_row_stride, void* out, int out_dtype, long long out_row_stride,
                          int n_rows, int width, int groups, float eps, int gate_rule, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_rows >= 0 && width > 0 && groups > 0 && width % groups == 0 && (long long)n_rows * groups < (1ll << 31),
           "rmsnorm: bad sizes rows=%d width=%d groups=%d", n_rows, width, groups);
  BT_CHECK((x_dtype == kF32 || x_dtype == kBF16) && (out_dtype == kF32 || out_dtype == kBF16) &&
           (gate == nullptr || gate_dtype == kF32 || gate_dtype == kBF16), "rmsnorm: unknown dtype");
  if (n_rows == 0) return 0;
  const bool gate_bf16 = gate != nullptr && gate_dtype == kBF16;
  if (x_dtype == kF32 && !gate_bf16)
    return launch_rmsnorm((const float*)x, x_row_stride, weight, (const float*)gate, gate_row_stride, out, out_row_stride,
                          n_rows, width, groups, eps, out_dtype, gate_rule, stream);
  if (x_dtype == kF32)
    return launch_rmsnorm((const float*)x, x_row_stride, weight, (const __nv_bfloat16*)gate, gate_row_stride, out,
                          out_row_stride, n_rows, width, groups, eps, out_dtype, gate_rule, stream);
  if (!gate_bf16)
    return launch_rmsnorm((const __nv_bfloat16*)x, x_row_stride, weight, (const float*)gate, gate_row_stride, out,
                          out_row_stride, n_rows, width, groups, eps, out_dtype, gate_rule, stream);
  return launch_rmsnorm((const __nv_bfloat16*)x, x_row_stride, weight, (const __nv_bfloat16*)gate, gate_row_stride, out,
                        out_row_stride, n_rows, width, groups, eps, out_dtype, gate_rule, stream);
}

extern "C" int bt_rotary_interleaved(const void* src, long long src_row_stride, int src_vec_stride, void* dst,
                                     long long dst_row_stride, int dst_vec_stride, const int* positions,
                                     const float* inv_freq, int n_tokens, int n_vecs, int len, int dims, int dtype,
                                     cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_vecs > 0 && len > 0 && dims >= 0 && dims <= len && dims % 2 == 0,
           "rotary_interleaved: bad sizes vectors=%d len=%d dims=%d", n_vecs, len, dims);
  if (n_tokens == 0) return 0;
  if (dtype == kF32)
    BT_PDL_OK("rotary_interleaved", launch_pdl(rotary_interleaved_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, 1,
                                               (const float*)src, src_row_stride, src_vec_stride, (float*)dst,
                                               dst_row_stride, dst_vec_stride, positions, inv_freq, n_vecs, len, dims));
  else if (dtype == kBF16)
    BT_PDL_OK("rotary_interleaved",
              launch_pdl(rotary_interleaved_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, stream, 1,
                         (const __nv_bfloat16*)src, src_row_stride, src_vec_stride, (__nv_bfloat16*)dst, dst_row_stride,
                         dst_vec_stride, positions, inv_freq, n_vecs, len, dims));
  else
    return fail("rotary_interleaved: unknown dtype %d", dtype);
  return 0;
}

extern "C" int bt_gated_activation(const void* x, void* out, long long n_rows, int inner, int act, float limit,
                                   int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_rows >= 0 && inner > 0, "gated_activation: bad sizes rows=%lld inner=%d", n_rows, inner);
  if (n_rows == 0) return 0;
  const long long total = n_rows * inner;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (dtype == kF32)
    BT_PDL_OK("gated_activation", launch_pdl(gated_activation_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1,
                                             (const float*)x, (float*)out, n_rows, inner, act, limit));
  else if (dtype == kBF16 && inner % 8 == 0 && (unsigned long long)x % 16 == 0 && (unsigned long long)out % 16 == 0) {
    const long long pieces = total / 8;
    const int b8 = (int)((pieces + 255) / 256 < 148 * 16 ? (pieces + 255) / 256 : 148 * 16);
    BT_PDL_OK("gated_activation", launch_pdl(gated_activation_bf16x8_kernel, dim3(b8), dim3(256), 0, stream, 1,
                                             (const __nv_bfloat16*)x, (__nv_bfloat16*)out, n_rows, inner, act, limit));
  } else if (dtype == kBF16)
    BT_PDL_OK("gated_activation", launch_pdl(gated_activation_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, 1,
                                             (const __nv_bfloat16*)x, (__nv_bfloat16*)out, n_rows, inner, act, limit));
  else
    return fail("gated_activation: unknown dtype %d", dtype);
  return 0;
}

extern "C" int bt_scale(float* x, long long n, float scale, cudaStream_t stream) {
  using namespace bt;
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  BT_PDL_OK("scale", launch_pdl(scale_kernel, dim3(blocks), dim3(256), 0, stream, 1, x, n, scale));
  return 0;
}

extern "C" int bt_add_vector(float* x, const float* vec, long long n_rows, int width, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_rows >= 0 && width > 0, "add_vector: bad sizes rows=%lld width=%d", n_rows, width);
  if (n_rows == 0) return 0;
  const long long total = n_rows * width;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  BT_PDL_OK("add_vector", launch_pdl(add_vector_kernel, dim3(blocks), dim3(256), 0, stream, 1, x, vec, n_rows, width));
  return 0;
}

extern "C" int bt_add_rows(float* x, const float* a, const float* b, const float* c, long long n, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n >= 0 && a != nullptr, "add_rows: bad arguments");
  if (n == 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  BT_PDL_OK("add_rows", launch_pdl(add_rows_kernel, dim3(blocks), dim3(256), 0, stream, 1, x, a, b, c, n));
  return 0;
}

namespace bt {

// stream_rows[r] += x[r] / sqrt(mean(x[r]^2) + eps) * weight: a sublayer's result, normed, joins the 32-bit stream.
// With next_out the row that the stream then holds is normed once more (next_weight) into next_out: the norm that
// opens the next sublayer, in the same pass over the row.
template <typename TOut>
__global__ void __launch_bounds__(128)
rmsnorm_add_kernel(const float* __restrict__ x, const float* __restrict__ weight, float* __restrict__ stream_rows,
                   const float* __restrict__ next_weight, TOut* __restrict__ next_out, int width, float eps, float factor) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const long long r = blockIdx.x;
  const float* src = x + r * width;
  float* dst = stream_rows + r * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(src[c], src[c], ss);
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
  float ss2 = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = fmaf(factor, src[c] * inv * weight[c], dst[c]);
    dst[c] = v;
    ss2 = fmaf(v, v, ss2);
  }
  if (next_out == nullptr) return;
  if (next_weight == nullptr) {       // the next sublayer reads the new row as it is, in its own element type
    for (int c = threadIdx.x; c < width; c += blockDim.x) next_out[r * width + c] = from_float<TOut>(dst[c]);
    return;
  }
  const float inv2 = 1.f / sqrtf(block_sum(ss2, scratch) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x)       // (a thread reads back what it wrote itself)
    next_out[r * width + c] = from_float<TOut>(dst[c] * inv2 * next_weight[c]);
}

// out[r] = a N(z) + b N(z^2) + c N(z^3) + e over a row z = x[r], powers element by element, N(v) = v / sqrt(mean(v^2) + eps);
// coef = (a, b, c, e).  32-bit throughout, rounded once.
template <typename T>
__global__ void __launch_bounds__(256)
polynorm_kernel(const T* __restrict__ x, const float* __restrict__ coef, T* __restrict__ out, int width, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const long long r = blockIdx.x;
  const T* src = x + r * width;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float z = to_float(src[c]), z2 = z * z;
    s2 += z2;
    s4 = fmaf(z2, z2, s4);
    s6 = fmaf(z2 * z, z2 * z, s6);
  }
  const float n = (float)width;
  const float i1 = coef[0] / sqrtf(block_sum(s2, scratch) / n + eps);
  const float i2 = coef[1] / sqrtf(block_sum(s4, scratch) / n + eps);
  const float i3 = coef[2] / sqrtf(block_sum(s6, scratch) / n + eps);
  const float shift = coef[3];
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float z = to_float(src[c]), z2 = z * z;
    out[r * width + c] = from_float<T>(fmaf(z, i1, fmaf(z2, i2, fmaf(z2 * z, i3, shift))));
  }
}

// dst[t, v, :] (32-bit) = src[t, v, :] with channel i < dims/2 paired with channel i + dims/2 and the pair turned by
// positions[t] * inv_freq[i]; channels from `dims` on pass; vectors from `scaled_from` on are multiplied by `scale`
// afterwards.  The `tail` channels that follow the vectors in a row are copied as they are.
template <typename T>
__global__ void __launch_bounds__(128)
rotary_half_kernel(const T* __restrict__ src, long long src_row_stride, float* __restrict__ dst, long long dst_row_stride,
                   const int* __restrict__ positions, const float* __restrict__ inv_freq, int n_vecs, int len, int dims,
                   int scaled_from, float scale, int tail) {
  pdl_trigger();
  pdl_wait();
  const long long t = blockIdx.x;
  const float pos = (float)positions[t];
  const int half = dims / 2, units = len - half;      // a unit: one pair, or one channel that passes
  const T* s_row = src + t * src_row_stride;
  float* d_row = dst + t * dst_row_stride;
  for (int i = threadIdx.x; i < n_vecs * units; i += blockDim.x) {
    const int v = i / units, u = i - v * units;
    const T* s = s_row + (long long)v * len;
    float* d = d_row + (long long)v * len;
    const float f = v >= scaled_from ? scale : 1.f;
    if (u < half) {
      float sn, cs;
      sincosf(pos * inv_freq[u], &sn, &cs);
      const float a = to_float(s[u]), b = to_float(s[u + half]);
      d[u] = (a * cs - b * sn) * f;
      d[u + half] = (b * cs + a * sn) * f;
    } else {
      d[half + u] = to_float(s[half + u]) * f;
    }
  }
  const int base = n_vecs * len;
  for (int i = threadIdx.x; i < tail; i += blockDim.x) d_row[base + i] = to_float(s_row[base + i]);
}

// out[t] = x[t] + (x[t - 1] - x[t]) * shift for the rows of a step, a sequence's rows one after another; the row before a
// sequence's first row of the step is state[slot] (zeros for a new sequence), which then becomes the sequence's last
// row.  A block a row; the block of a sequence's last row also does its first row, which reads the state, and writes the
// state afterwards, so that nothing reads what another block replaces.
template <typename TOut>
__global__ void __launch_bounds__(128)
token_shift_kernel(const float* __restrict__ x, const float* __restrict__ shift, float* __restrict__ state,
                   const int* __restrict__ slots, const int* __restrict__ seq_start, const int* __restrict__ token_seq,
                   TOut* __restrict__ out, int width) {
  pdl_trigger();
  pdl_wait();
  const long long t = blockIdx.x;
  const int seq = token_seq[t];
  const long long first = seq_start[seq], last = (long long)seq_start[seq + 1] - 1;
  float* kept = state + (long long)slots[seq] * width;
  if (t != first || t == last) {
    const float* cur = x + t * width;
    const float* prev = t == first ? kept : cur - width;
    for (int c = threadIdx.x; c < width; c += blockDim.x)
      out[t * width + c] = from_float<TOut>(fmaf(prev[c] - cur[c], shift[c], cur[c]));
  }
  if (t != last) return;
  if (first != last) {
    const float* cur = x + first * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x)
      out[first * width + c] = from_float<TOut>(fmaf(kept[c] - cur[c], shift[c], cur[c]));
  }
  const float* cur = x + last * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) kept[c] = cur[c];      // (a thread read kept[c] itself above)
}

}  // namespace bt

extern "C" int bt_token_shift(const float* x, const float* shift, float* state, const int* slots, const int* seq_start,
                              const int* token_seq, void* out, int out_dtype, long long n_rows, int width,
                              cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_rows >= 0 && n_rows < (1ll << 31) && width > 0, "token_shift: bad sizes rows=%lld width=%d", n_rows, width);
  if (n_rows == 0) return 0;
  if (out_dtype == kBF16)
    BT_PDL_OK("token_shift", launch_pdl(token_shift_kernel<__nv_bfloat16>, dim3((unsigned)n_rows), dim3(128), 0, stream, 1, x,
                                        shift, state, slots, seq_start, token_seq, (__nv_bfloat16*)out, width));
  else if (out_dtype == kF32)
    BT_PDL_OK("token_shift", launch_pdl(token_shift_kernel<float>, dim3((unsigned)n_rows), dim3(128), 0, stream, 1, x, shift,
                                        state, slots, seq_start, token_seq, (float*)out, width));
  else
    return fail("token_shift: unknown dtype %d", out_dtype);
  return 0;
}

extern "C" int bt_rmsnorm_add(const float* x, const float* weight, float* stream_rows, const float* next_weight,
                              void* next_out, int next_dtype, long long n_rows, int width, float eps, float factor,
                              cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_rows >= 0 && n_rows < (1ll << 31) && width > 0, "rmsnorm_add: bad sizes rows=%lld width=%d", n_rows, width);
  BT_CHECK(next_out == nullptr || next_dtype == kF32 || next_dtype == kBF16, "rmsnorm_add: the next rows need a known dtype");
  if (n_rows == 0) return 0;
  if (next_out != nullptr && next_dtype == kBF16)
    BT_PDL_OK("rmsnorm_add", launch_pdl(rmsnorm_add_kernel<__nv_bfloat16>, dim3((unsigned)n_rows), dim3(128), 0, stream, 1, x,
                                        weight, stream_rows, next_weight, (__nv_bfloat16*)next_out, width, eps, factor));
  else
    BT_PDL_OK("rmsnorm_add", launch_pdl(rmsnorm_add_kernel<float>, dim3((unsigned)n_rows), dim3(128), 0, stream, 1, x, weight,
                                        stream_rows, next_weight, (float*)next_out, width, eps, factor));
  return 0;
}

extern "C" int bt_polynorm(const void* x, const float* coef, void* out, long long n_rows, int width, float eps, int dtype,
                           cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_rows >= 0 && n_rows < (1ll << 31) && width > 0, "polynorm: bad sizes rows=%lld width=%d", n_rows, width);
  if (n_rows == 0) return 0;
  if (dtype == kF32)
    BT_PDL_OK("polynorm", launch_pdl(polynorm_kernel<float>, dim3((unsigned)n_rows), dim3(256), 0, stream, 1, (const float*)x,
                                     coef, (float*)out, width, eps));
  else if (dtype == kBF16)
    BT_PDL_OK("polynorm", launch_pdl(polynorm_kernel<__nv_bfloat16>, dim3((unsigned)n_rows), dim3(256), 0, stream, 1,
                                     (const __nv_bfloat16*)x, coef, (__nv_bfloat16*)out, width, eps));
  else
    return fail("polynorm: unknown dtype %d", dtype);
  return 0;
}

extern "C" int bt_rotary_half(const void* src, long long src_row_stride, int src_dtype, float* dst, long long dst_row_stride,
                              const int* positions, const float* inv_freq, int n_tokens, int n_vecs, int len, int dims,
                              int scaled_from, float scale, int tail, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_vecs > 0 && len > 0 && dims >= 0 && dims <= len && dims % 2 == 0 && tail >= 0,
           "rotary_half: bad sizes vectors=%d len=%d dims=%d", n_vecs, len, dims);
  if (n_tokens == 0) return 0;
  if (src_dtype == kF32)
    BT_PDL_OK("rotary_half", launch_pdl(rotary_half_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, 1, (const float*)src,
                                        src_row_stride, dst, dst_row_stride, positions, inv_freq, n_vecs, len, dims,
                                        scaled_from, scale, tail));
  else if (src_dtype == kBF16)
    BT_PDL_OK("rotary_half", launch_pdl(rotary_half_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, stream, 1,
                                        (const __nv_bfloat16*)src, src_row_stride, dst, dst_row_stride, positions, inv_freq,
                                        n_vecs, len, dims, scaled_from, scale, tail));
  else
    return fail("rotary_half: unknown dtype %d", src_dtype);
  return 0;
}
