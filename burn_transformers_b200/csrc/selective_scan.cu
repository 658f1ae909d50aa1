// A selective state-space scan: per channel c and state index n a 32-bit state that every token decays and feeds,
//
//     dt[t, c] = softplus(sum_r W_dt[c, r] * low[t, r] + b_dt[c])                       (selective_scan_dt)
//     S[c, n] <- exp(dt[t, c] * A[c, n]) * S[c, n] + dt[t, c] * x[t, c] * B[t, n]       A = -exp(A_log)
//     y[t, c]  = (sum_n S[c, n] * C[t, n] + D[c] * x[t, c]) * z[t, c] * sigmoid(z[t, c]) * out_scale
//
// B and C are channels of the step's rows `low` (one vector per token, shared by all channels); x and z are channels
// of other rows.  Step sizes, decays, the state and all sums are 32-bit.  A channel belongs to LANES adjacent lanes,
// each with NS of the `n_state` indices in registers for all tokens of the step; their partial sums meet by shuffles.
// The tokens of a run are staged in shared memory TT at a time.  state: [slots][channels][n_state].
//
// A long run is cut into pieces of `piece` tokens that run side by side.  A first launch (ENDS) runs every piece but a
// sequence's last from a zero state and leaves, per channel, what it ends with, E[n], and the sum of its step sizes, d;
// the state after the piece is then exp(A[n] d) * (state before it) + E[n], since the recurrence is linear in the state
// and its decays multiply to exp(A[n] * sum dt).  The second launch gives every piece its own block, which first walks
// the earlier pieces' (E, d) from the sequence's stored state to its own start and then runs its tokens as the single
// run would; the last piece writes the state back.  `ends`: [pieces of the step][channels][n_state + 1], where the
// pieces of sequence s begin at first_row(s) / piece + s.
#include "common.cuh"

namespace bt {

constexpr int SS_TT = 16;        // tokens staged at a time
constexpr int SS_THREADS = 128;
constexpr int SS_WS = 257;       // floats between the rank indices of the step sizes' weights in shared memory

__device__ __forceinline__ float ss_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// exp(d * a) for the decay of a step, a <= 0.  With bfloat16 rows the exponent is formed in base 2 (a_scaled = a log2 e)
// and raised by the special-function unit (2 units in the last place); 32-bit rows take the library's exp.
template <typename T>
__device__ __forceinline__ float ss_decay(float d, float a_scaled) {
  if constexpr (sizeof(T) == 2) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(d * a_scaled));
    return y;
  } else {
    return expf(d * a_scaled);
  }
}

// dt[t, c], a block: 256 channels x SS_TT tokens; W_dt's rows of these channels lie transposed in shared memory
template <typename T>
__global__ void __launch_bounds__(256)
selective_scan_dt_kernel(const T* __restrict__ low, long long low_row_stride, const float* __restrict__ w_dt,
                         const float* __restrict__ b_dt, float* __restrict__ dt, long long n_tokens, int channels,
                         int rank) {
  extern __shared__ float sm[];
  float* low_s = sm;                       // [rank][SS_TT]
  float* w_s = low_s + rank * SS_TT;       // [rank][SS_WS]: padded, so that the transposing stores spread over the banks
  pdl_trigger();
  const int c0 = blockIdx.x * 256, c = c0 + threadIdx.x;
  for (int i = threadIdx.x; i < rank * 256; i += 256) {
    const int cl = i / rank, r = i - cl * rank;
    w_s[r * SS_WS + cl] = c0 + cl < channels ? w_dt[(long long)(c0 + cl) * rank + r] : 0.f;
  }
  const float bias = c < channels ? b_dt[c] : 0.f;
  pdl_wait();
  for (long long t0 = (long long)blockIdx.y * SS_TT; t0 < n_tokens; t0 += (long long)gridDim.y * SS_TT) {
    const int nt = (int)min((long long)SS_TT, n_tokens - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < SS_TT * rank; i += 256) {
      const int t = i / rank, r = i - t * rank;
      low_s[r * SS_TT + t] = t < nt ? to_float(low[(t0 + t) * low_row_stride + r]) : 0.f;
    }
    __syncthreads();
    // a thread a channel: its weight once per rank index against the SS_TT tokens' numbers, read four at a time
    float acc[SS_TT];
#pragma unroll
    for (int t = 0; t < SS_TT; ++t) acc[t] = bias;
    for (int r = 0; r < rank; ++r) {
      const float w = w_s[r * SS_WS + threadIdx.x];
#pragma unroll
      for (int t4 = 0; t4 < SS_TT / 4; ++t4) {
        const float4 x = *reinterpret_cast<const float4*>(low_s + r * SS_TT + t4 * 4);
        acc[t4 * 4 + 0] = fmaf(w, x.x, acc[t4 * 4 + 0]);
        acc[t4 * 4 + 1] = fmaf(w, x.y, acc[t4 * 4 + 1]);
        acc[t4 * 4 + 2] = fmaf(w, x.z, acc[t4 * 4 + 2]);
        acc[t4 * 4 + 3] = fmaf(w, x.w, acc[t4 * 4 + 3]);
      }
    }
    if (c < channels) {
#pragma unroll
      for (int t = 0; t < SS_TT; ++t)
        if (t < nt) dt[(t0 + t) * channels + c] = ss_softplus(acc[t]);
    }
  }
}

template <typename T, int NS, int LANES, bool ENDS>
__global__ void __launch_bounds__(SS_THREADS)
selective_scan_kernel(const T* __restrict__ x, long long x_row_stride, const T* __restrict__ z, long long z_row_stride,
                      const float* __restrict__ dt, const T* __restrict__ low, long long low_row_stride, int b_off,
                      int c_off, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                      float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ seq_start,
                      T* __restrict__ out, long long out_row_stride, int channels, int n_state, float out_scale, int piece,
                      float* __restrict__ ends, int stage) {
  constexpr int CPB = SS_THREADS / LANES;      // channels per block
  extern __shared__ float sm[];
  float* bc_s = sm;                            // [stage][2 * n_state]
  float* dt_s = bc_s + stage * 2 * n_state;    // [stage][CPB]
  float* x_s = dt_s + stage * CPB;
  float* z_s = x_s + stage * CPB;
  pdl_trigger();
  const int seq = blockIdx.y, c_local = threadIdx.x / LANES, part = threadIdx.x % LANES;
  const int c = blockIdx.x * CPB + c_local;
  const bool owns = c < channels;
  const int n0 = part * NS;
  float a[NS], s[NS];      // a: A = -exp(A_log), times log2 e where the decays are raised in base 2
#pragma unroll
  for (int i = 0; i < NS; ++i)
    a[i] = owns && n0 + i < n_state ? -expf(a_log[(long long)c * n_state + n0 + i]) * (sizeof(T) == 2 ? 1.4426950408889634f : 1.f)
                                    : 0.f;
  const float skip = owns ? d_skip[c] : 0.f;
  pdl_wait();
  const int first = seq_start[seq], n_all = seq_start[seq + 1] - first;
  // this block's piece of the run: tokens [t_lo, t_hi); the whole run when piece == 0
  const int n_pieces = piece > 0 ? (n_all + piece - 1) / piece : 1;
  const int my_piece = piece > 0 ? (int)blockIdx.z : 0;
  if (my_piece >= n_pieces - (ENDS ? 1 : 0)) return;
  const int t_lo = my_piece * piece, t_hi = piece > 0 ? min(n_all, t_lo + piece) : n_all;
  const bool last_piece = my_piece == n_pieces - 1;
  const long long es = (long long)channels * (n_state + 1);
  float* e_base = piece > 0 ? ends + ((long long)(first / piece + seq)) * es + (long long)(owns ? c : 0) * (n_state + 1) : nullptr;
  float* s_base = state + ((long long)slots[seq] * channels + (owns ? c : 0)) * n_state;
  float dt_sum = 0.f;
#pragma unroll
  for (int i = 0; i < NS; ++i) s[i] = !ENDS && owns && n0 + i < n_state ? s_base[n0 + i] : 0.f;
  if (!ENDS && owns) {
    for (int j = 0; j < my_piece; ++j) {
      const float* e = e_base + (long long)j * es;
      const float d = e[n_state];
#pragma unroll
      for (int i = 0; i < NS; ++i)
        if (n0 + i < n_state) s[i] = fmaf(ss_decay<T>(d, a[i]), s[i], e[n0 + i]);
    }
  }
  // B and C of a token as 16-byte pieces where the lane's state indices are whole pieces of a row
  const bool vec = (n_state & 3) == 0 && n0 + NS <= n_state;
  for (int t0 = t_lo; t0 < t_hi; t0 += stage) {
    const int nt = min(stage, t_hi - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * 2 * n_state; i += SS_THREADS) {
      const int t = i / (2 * n_state), n = i - t * 2 * n_state;
      const T* row = low + (long long)(first + t0 + t) * low_row_stride;
      bc_s[i] = to_float(n < n_state ? row[b_off + n] : row[c_off + n - n_state]);
    }
    for (int i = threadIdx.x; i < nt * CPB; i += SS_THREADS) {
      const int t = i / CPB, cl = i - t * CPB, cc = blockIdx.x * CPB + cl;
      const long long r = first + t0 + t;
      const bool in = cc < channels;
      dt_s[i] = in ? dt[r * channels + cc] : 0.f;
      x_s[i] = in ? to_float(x[r * x_row_stride + cc]) : 0.f;
      z_s[i] = in ? to_float(z[r * z_row_stride + cc]) : 0.f;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float d = dt_s[t * CPB + c_local], xv = x_s[t * CPB + c_local];
      const float dx = d * xv;
      const float* bt_ = bc_s + t * 2 * n_state + n0;
      const float* ct_ = bt_ + n_state;
      float y = 0.f;
      if (vec) {
#pragma unroll
        for (int i4 = 0; i4 < NS / 4; ++i4) {
          const float4 b4 = *reinterpret_cast<const float4*>(bt_ + 4 * i4), c4 = *reinterpret_cast<const float4*>(ct_ + 4 * i4);
          const float bs[4] = {b4.x, b4.y, b4.z, b4.w}, cs[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int i = 4 * i4 + k;
            s[i] = fmaf(ss_decay<T>(d, a[i]), s[i], dx * bs[k]);
            y = fmaf(s[i], cs[k], y);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < NS; ++i) {
          if (n0 + i < n_state) {
            s[i] = fmaf(ss_decay<T>(d, a[i]), s[i], dx * bt_[i]);
            y = fmaf(s[i], ct_[i], y);
          }
        }
      }
      if (!ENDS) {
#pragma unroll
        for (int o = 1; o < LANES; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      }
      dt_sum += d;
      if (ENDS) continue;
      if (owns && part == 0) {
        const float zv = z_s[t * CPB + c_local];
        const float r = (y + skip * xv) * (zv / (1.f + expf(-zv))) * out_scale;
        out[(long long)(first + t0 + t) * out_row_stride + c] = from_float<T>(r);
      }
    }
  }
  if (ENDS) {
    if (owns) {
      float* e = e_base + (long long)my_piece * es;
#pragma unroll
      for (int i = 0; i < NS; ++i)
        if (n0 + i < n_state) e[n0 + i] = s[i];
      if (part == 0) e[n_state] = dt_sum;
    }
    return;
  }
  if (owns && last_piece) {
#pragma unroll
    for (int i = 0; i < NS; ++i)
      if (n0 + i < n_state) s_base[n0 + i] = s[i];
  }
}

template <typename T>
static int launch_selective_scan(const T* x, long long xs, const T* z, long long zs, const float* dt, const T* low,
                                 long long ls, int b_off, int c_off, const float* a_log, const float* d_skip, float* state,
                                 const int* slots, const int* seq_start, T* out, long long os, int n_seqs, int channels,
                                 int n_state, float out_scale, int piece, int max_pieces, float* ends,
                                 cudaStream_t stream) {
  int ns, lanes;
  if (n_state <= 16) { ns = 4; lanes = 4; }
  else if (n_state <= 32) { ns = 8; lanes = 4; }
  else if (n_state <= 64) { ns = 16; lanes = 4; }
  else if (n_state <= 128) { ns = 16; lanes = 8; }
  else if (n_state <= 256) { ns = 16; lanes = 16; }
  else { ns = 16; lanes = 32; }
  BT_CHECK(n_state <= 512, "selective_scan: %d state indices a channel; the kernel takes up to 512", n_state);
  const int cpb = SS_THREADS / lanes;
  const dim3 grid((channels + cpb - 1) / cpb, n_seqs, piece > 0 ? max_pieces : 1);
  const int stage = n_state <= 64 ? 2 * SS_TT : SS_TT;      // tokens staged in shared memory at a time
  const size_t smem = sizeof(float) * ((size_t)stage * 2 * n_state + 3 * (size_t)stage * cpb);
#define BT_SS(NS, LANES)                                                                                              \
  do {                                                                                                                \
    if (smem > 48 * 1024)                                                                                             \
      BT_CHECK(cudaFuncSetAttribute(selective_scan_kernel<T, NS, LANES, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                    (int)smem) == cudaSuccess &&                                                      \
               cudaFuncSetAttribute(selective_scan_kernel<T, NS, LANES, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                    (int)smem) == cudaSuccess, "selective_scan: cannot reserve %zu bytes of shared memory", smem); \
    if (piece > 0)                                                                                                    \
      BT_PDL_OK("selective_scan", launch_pdl(selective_scan_kernel<T, NS, LANES, true>, grid, dim3(SS_THREADS), smem, \
                                             stream, 1, x, xs, z, zs, dt, low, ls, b_off, c_off, a_log, d_skip, state, \
                                             slots, seq_start, out, os, channels, n_state, out_scale, piece, ends,     \
                                             stage));                                                                 \
    BT_PDL_OK("selective_scan", launch_pdl(selective_scan_kernel<T, NS, LANES, false>, grid, dim3(SS_THREADS), smem,   \
                                           stream, 1, x, xs, z, zs, dt, low, ls, b_off, c_off, a_log, d_skip, state,   \
                                           slots, seq_start, out, os, channels, n_state, out_scale, piece, ends,       \
                                           stage));                                                                   \
  } while (0)
  if (ns == 4) BT_SS(4, 4);
  else if (ns == 8) BT_SS(8, 4);
  else if (lanes == 4) BT_SS(16, 4);
  else if (lanes == 8) BT_SS(16, 8);
  else if (lanes == 16) BT_SS(16, 16);
  else BT_SS(16, 32);
#undef BT_SS
  return 0;
}

}  // namespace bt

// dt [tokens, channels] 32-bit from the first `rank` channels of the rows of low
extern "C" int bt_selective_scan_dt(const void* low, long long low_row_stride, const float* w_dt, const float* b_dt,
                                    float* dt, long long n_tokens, int channels, int rank, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(channels > 0 && rank > 0 && rank <= 160 && n_tokens >= 0,
           "selective_scan_dt: bad sizes channels=%d rank=%d (at most 160)", channels, rank);
  if (n_tokens == 0) return 0;
  const size_t smem = sizeof(float) * ((size_t)rank * SS_WS + (size_t)SS_TT * rank);
  const long long tiles = (n_tokens + SS_TT - 1) / SS_TT;
  const long long col_blocks = (channels + 255) / 256, want_rows = (4 * 148 + col_blocks - 1) / col_blocks;
  const dim3 grid((unsigned)col_blocks, (unsigned)(tiles < want_rows ? tiles : want_rows));      // (about four blocks an SM)
#define BT_SSD(T)                                                                                                     \
  do {                                                                                                                \
    auto kern = selective_scan_dt_kernel<T>;                                                                          \
    if (smem > 48 * 1024)                                                                                             \
      BT_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess,     \
               "selective_scan_dt: cannot reserve %zu bytes of shared memory", smem);                                 \
    BT_PDL_OK("selective_scan_dt", launch_pdl(kern, grid, dim3(256), smem, stream, 1, (const T*)low, low_row_stride, w_dt, \
                                              b_dt, dt, n_tokens, channels, rank));                                    \
  } while (0)
  if (dtype == kF32) BT_SSD(float);
  else if (dtype == kBF16) BT_SSD(__nv_bfloat16);
  else return fail("selective_scan_dt: unknown dtype %d", dtype);
#undef BT_SSD
  return 0;
}

// x, z, out: first channel of [tokens, channels] views; low: the rows that hold B at b_off and C at c_off.
// piece > 0: runs are cut into pieces of `piece` tokens (a multiple of 16), none has more than max_pieces, and `ends`
// holds (n_tokens / piece + n_seqs + 1) * channels * (n_state + 1) floats; piece == 0: a block walks a whole run.
extern "C" int bt_selective_scan(const void* x, long long x_row_stride, const void* z, long long z_row_stride,
                                 const float* dt, const void* low, long long low_row_stride, int b_off, int c_off,
                                 const float* a_log, const float* d_skip, float* state, const int* slots,
                                 const int* seq_start, void* out, long long out_row_stride, int n_seqs, int channels,
                                 int n_state, float out_scale, int piece, int max_pieces, float* ends, int dtype,
                                 cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(piece == 0 || (piece % SS_TT == 0 && max_pieces > 0 && max_pieces <= 65535 && ends != nullptr),
           "selective_scan: pieces of %d tokens (a multiple of %d), at most %d a run, need scratch", piece, SS_TT, max_pieces);
  BT_CHECK(channels > 0 && n_state > 0 && n_seqs >= 0 && n_seqs <= 65535, "selective_scan: bad sizes seqs=%d channels=%d "
           "state=%d", n_seqs, channels, n_state);
  if (n_seqs == 0) return 0;
  if (dtype == kF32)
    return launch_selective_scan((const float*)x, x_row_stride, (const float*)z, z_row_stride, dt, (const float*)low,
                                 low_row_stride, b_off, c_off, a_log, d_skip, state, slots, seq_start, (float*)out,
                                 out_row_stride, n_seqs, channels, n_state, out_scale, piece, max_pieces, ends, stream);
  if (dtype == kBF16)
    return launch_selective_scan((const __nv_bfloat16*)x, x_row_stride, (const __nv_bfloat16*)z, z_row_stride, dt,
                                 (const __nv_bfloat16*)low, low_row_stride, b_off, c_off, a_log, d_skip, state, slots,
                                 seq_start, (__nv_bfloat16*)out, out_row_stride, n_seqs, channels, n_state, out_scale, piece,
                                 max_pieces, ends, stream);
  return fail("selective_scan: unknown dtype %d", dtype);
}
