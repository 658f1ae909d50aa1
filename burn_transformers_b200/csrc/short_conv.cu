// A short causal convolution over time on every channel of the step's rows, with the sequence's last taps - 1 inputs
// kept as 32-bit state between steps:
//
//     y[t, c] = act(bias[c] + sum_j w[c, j] * u[t - taps + 1 + j, c])        j = 0 .. taps - 1
//
// u before the sequence's first token is zero (a new sequence finds zeros in its state).  Token t of a sequence that
// brings n tokens this step reads inputs of this step where t - d >= 0 and state[taps - 1 + (t - d)] otherwise.
// state: [slots][taps - 1][channels], the newest input last.  Sums are 32-bit, in the order of j.
//
// Two forms: channel by channel (optionally x * sigmoid(x) on the result), and a warp per (token, run of `group`
// channels) that also divides the run by its root mean square (a head's query or key) and can leave the undivided
// result of the runs from `raw_first_group` on in a second place (keys that are also the values).
// A third kernel moves the state on; it runs after the convolution (which reads the old state).
#include "common.cuh"

namespace bt {

constexpr int SC_MAX_TAPS = 16;

__device__ __forceinline__ float sc_silu(float x) { return x / (1.f + expf(-x)); }

template <typename TIn>
__device__ __forceinline__ float short_conv_at(const TIn* __restrict__ src, long long src_row_stride,
                                               const float* __restrict__ w, const float* __restrict__ bias,
                                               const float* __restrict__ state_row, int channels, int taps, long long t,
                                               int r, int c) {
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int d = taps - 1 - j, idx = r - d;
    const float u = idx >= 0 ? to_float(src[(t - d) * src_row_stride + c])
                             : state_row[(long long)(taps - 1 + idx) * channels + c];
    acc = fmaf(w[(long long)c * taps + j], u, acc);
  }
  return acc;
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
short_conv_kernel(const TIn* __restrict__ src, long long src_row_stride, const float* __restrict__ w,
                  const float* __restrict__ bias, const float* __restrict__ state, const int* __restrict__ slots,
                  const int* __restrict__ seq_start, const int* __restrict__ token_seq, TOut* __restrict__ out,
                  long long out_row_stride, long long n_tokens, int channels, int taps, int act) {
  pdl_trigger();
  pdl_wait();
  const long long total = n_tokens * channels;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / channels;
    const int c = (int)(i - t * channels);
    const int seq = token_seq[t];
    const int r = (int)(t - seq_start[seq]);
    const float* state_row = state + (long long)slots[seq] * (taps - 1) * channels;
    float y = short_conv_at(src, src_row_stride, w, bias, state_row, channels, taps, t, r, c);
    if (act == 1) y = sc_silu(y);
    out[t * out_row_stride + c] = from_float<TOut>(y);
  }
}

template <typename TIn, typename TOut, int NV>
__global__ void __launch_bounds__(128)
short_conv_norm_kernel(const TIn* __restrict__ src, long long src_row_stride, const float* __restrict__ w,
                       const float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ seq_start,
                       const int* __restrict__ token_seq, TOut* __restrict__ out, long long out_row_stride,
                       TOut* __restrict__ raw_out, long long raw_row_stride, int raw_first_group, long long items,
                       int groups, int group, int taps, float eps) {
  pdl_trigger();
  pdl_wait();
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= items) return;
  const int lane = threadIdx.x & 31;
  const long long t = item / groups;
  const int g = (int)(item - t * groups);
  const int channels = groups * group;
  const int seq = token_seq[t];
  const int r = (int)(t - seq_start[seq]);
  const float* state_row = state + (long long)slots[seq] * (taps - 1) * channels;
  float y[NV], ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    y[i] = c < group ? short_conv_at(src, src_row_stride, w, (const float*)nullptr, state_row, channels, taps, t, r,
                                     g * group + c) : 0.f;
    ss = fmaf(y[i], y[i], ss);
  }
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)group + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < group) {
      out[t * out_row_stride + g * group + c] = from_float<TOut>(y[i] * inv);
      if (raw_out && g >= raw_first_group)
        raw_out[t * raw_row_stride + (g - raw_first_group) * group + c] = from_float<TOut>(y[i]);
    }
  }
}

// state[slot] <- the last taps - 1 inputs of the sequence after this step
template <typename TIn>
__global__ void __launch_bounds__(256)
short_conv_state_kernel(const TIn* __restrict__ src, long long src_row_stride, float* __restrict__ state,
                        const int* __restrict__ slots, const int* __restrict__ seq_start, int n_seqs, int channels,
                        int taps) {
  pdl_trigger();
  pdl_wait();
  const int keep = taps - 1;
  const long long total = (long long)n_seqs * channels;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int seq = (int)(i / channels), c = (int)(i - (long long)seq * channels);
    const int first = seq_start[seq], n_new = seq_start[seq + 1] - first;
    float* row = state + (long long)slots[seq] * keep * channels + c;
    float kept[SC_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < SC_MAX_TAPS; ++k) {
      if (k < keep) {
        const int r = n_new - keep + k;
        kept[k] = r >= 0 ? to_float(src[(long long)(first + r) * src_row_stride + c]) : row[(long long)(keep + r) * channels];
      }
    }
#pragma unroll
    for (int k = 0; k < SC_MAX_TAPS; ++k)
      if (k < keep) row[(long long)k * channels] = kept[k];
  }
}

static inline int sc_blocks(long long total) {
  const long long want = (total + 255) / 256;
  return (int)(want < 148 * 16 ? (want > 0 ? want : 1) : 148 * 16);
}

template <typename T>
static int launch_short_conv(const T* src, long long src_row_stride, const float* w, const float* bias, float* state,
                             const int* slots, const int* seq_start, const int* token_seq, void* out,
                             long long out_row_stride, int out_dtype, void* raw_out, long long raw_row_stride,
                             int raw_first_group, long long n_tokens, int n_seqs, int channels, int taps, int act,
                             int group, float eps, cudaStream_t stream) {
  if (group > 0) {
    const int groups = channels / group;
    const long long items = n_tokens * groups;
    const dim3 grid((unsigned)((items + 3) / 4));
#define BT_SCN(TOUT, NV)                                                                                             \
  BT_PDL_OK("short_conv_norm", launch_pdl(short_conv_norm_kernel<T, TOUT, NV>, grid, dim3(128), 0, stream, 1, src,    \
                                          src_row_stride, w, (const float*)state, slots, seq_start, token_seq,         \
                                          (TOUT*)out, out_row_stride, (TOUT*)raw_out, raw_row_stride, raw_first_group, \
                                          items, groups, group, taps, eps))
    if (out_dtype == kF32) {
      if (group <= 64) BT_SCN(float, 2); else if (group <= 128) BT_SCN(float, 4); else BT_SCN(float, 8);
    } else {
      if (group <= 64) BT_SCN(__nv_bfloat16, 2); else if (group <= 128) BT_SCN(__nv_bfloat16, 4); else BT_SCN(__nv_bfloat16, 8);
    }
#undef BT_SCN
  } else {
    const dim3 grid(sc_blocks(n_tokens * channels));
    if (out_dtype == kF32)
      BT_PDL_OK("short_conv", launch_pdl(short_conv_kernel<T, float>, grid, dim3(256), 0, stream, 1, src, src_row_stride, w,
                                         bias, (const float*)state, slots, seq_start, token_seq, (float*)out,
                                         out_row_stride, n_tokens, channels, taps, act));
    else
      BT_PDL_OK("short_conv", launch_pdl(short_conv_kernel<T, __nv_bfloat16>, grid, dim3(256), 0, stream, 1, src,
                                         src_row_stride, w, bias, (const float*)state, slots, seq_start, token_seq,
                                         (__nv_bfloat16*)out, out_row_stride, n_tokens, channels, taps, act));
  }
  if (taps > 1)
    BT_PDL_OK("short_conv_state", launch_pdl(short_conv_state_kernel<T>, dim3(sc_blocks((long long)n_seqs * channels)),
                                             dim3(256), 0, stream, 1, src, src_row_stride, state, slots, seq_start, n_seqs,
                                             channels, taps));
  return 0;
}

}  // namespace bt

// src: the first of `channels` adjacent channels of the step's rows; w [channels][taps] and bias [channels] 32-bit.
// group == 0: out = act(conv) channel by channel (act 1: x * sigmoid(x)).  group > 0: every run of `group` channels is
// divided by its root mean square (eps inside the root; no bias, no act) and, with raw_out, the runs from
// raw_first_group on are also left undivided at raw_out.  Afterwards the state holds the sequences' newest inputs.
extern "C" int bt_short_conv(const void* src, long long src_row_stride, int src_dtype, const float* w, const float* bias,
                             float* state, const int* slots, const int* seq_start, const int* token_seq, void* out,
                             long long out_row_stride, int out_dtype, void* raw_out, long long raw_row_stride,
                             int raw_first_group, long long n_tokens, int n_seqs, int channels, int taps, int act, int group,
                             float eps, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(channels > 0 && taps >= 1 && taps <= SC_MAX_TAPS && n_tokens >= 0 && n_seqs >= 0,
           "short_conv: bad sizes channels=%d taps=%d (at most %d)", channels, taps, SC_MAX_TAPS);
  BT_CHECK(group == 0 || (group > 0 && group <= 256 && channels % group == 0 && bias == nullptr && act == 0),
           "short_conv: runs of %d channels (at most 256, a divisor of %d, without bias or activation)", group, channels);
  BT_CHECK((src_dtype == kF32 || src_dtype == kBF16) && (out_dtype == kF32 || out_dtype == kBF16), "short_conv: unknown dtype");
  if (n_tokens == 0 || n_seqs == 0) return 0;
  if (src_dtype == kF32)
    return launch_short_conv((const float*)src, src_row_stride, w, bias, state, slots, seq_start, token_seq, out,
                             out_row_stride, out_dtype, raw_out, raw_row_stride, raw_first_group, n_tokens, n_seqs, channels,
                             taps, act, group, eps, stream);
  return launch_short_conv((const __nv_bfloat16*)src, src_row_stride, w, bias, state, slots, seq_start, token_seq, out,
                           out_row_stride, out_dtype, raw_out, raw_row_stride, raw_first_group, n_tokens, n_seqs, channels,
                           taps, act, group, eps, stream);
}
