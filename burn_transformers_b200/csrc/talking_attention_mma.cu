// Windowed softmax attention whose heads talk before the softmax (see talking_attention.cu for the equations), for
// bfloat16 rows on tensor cores.  Scores, their cap, bias and mixing, the softmax and the accumulators are 32-bit; the
// products q . k and weights x values take bfloat16 operands, and a weight enters its product as the sum of two
// bfloat16 numbers (the rounded weight and what the rounding dropped), so that it keeps 16 bits of mantissa.
//
// A block is 16 query tokens of one sequence with ALL heads, a warp a head.  Per tile of 32 keys: warp g multiplies its
// head's queries with the tile's keys (mma.sync, 16 x 32 scores in the accumulators), caps and biases them and leaves
// them in shared memory, every lane its own accumulators as 16-byte pieces; after a barrier warp h sums the heads'
// planes with row h of `talk`, lane by lane in the same layout, so that the weights pass from the accumulators to the
// value product's operand inside registers.  Key and value tiles
// (per key head, shared by its query heads) come through two cp.async buffers from the step's own rows or the pages.
// A step that brings at most 16 tokens a sequence (a decode step is the same block with one live row) may be cut over
// the keys: block b of `n_split` takes every n_split-th tile and leaves its running maximum, sum and accumulators in
// `parts`, and a second kernel joins them.
#include "decode_mma.cuh"

namespace bt {

constexpr int TM_BQ = 16, TM_KT = 32, TM_PAD = 8;

struct TalkingArgs {
  const __nv_bfloat16 *q, *gate;
  __nv_bfloat16* out;
  long long q_row, gate_row, out_row;
  KvView kv;
  const int *seq_start, *past_len;
  const float *temp, *slope, *talk;
  int n_heads, n_kv_heads, head_dim;
  float scale, cap, out_scale;
  int window;
  int n_split, max_new;     // n_split > 1: grid.x blocks share the key tiles of a sequence's (single) tile of queries
  float* parts;             // [seqs][n_split][heads][max_new][head_dim + 2]: accumulators, maximum (base 2), sum
};

__device__ __forceinline__ void tm_cp_async16(unsigned dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

static size_t tm_smem(int H, int G, int dp) {
  return (size_t)2 * TM_BQ * (H * dp + TM_PAD) + (size_t)2 * 2 * 2 * G * TM_KT * (dp + TM_PAD) +
         sizeof(float) * ((size_t)H * TM_BQ * TM_KT + (size_t)H * H);
}

// NP: 16-channel pieces of a head (head_dim <= 16 NP); WB: the most warps of a block
template <int NP, int WB>
__global__ void __launch_bounds__(32 * WB) talking_attention_mma_kernel(TalkingArgs p) {
  extern __shared__ __align__(16) unsigned char tm_raw[];
  constexpr float LOG2E = 1.4426950408889634f;
  constexpr int dp = 16 * NP, ldk = dp + TM_PAD, NT = TM_KT / 8;
  const int H = p.n_heads, G = p.n_kv_heads, D = p.head_dim;
  const int ldq = H * dp + TM_PAD;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(tm_raw);      // [16][ldq]
  __nv_bfloat16* k_s = q_s + TM_BQ * ldq;                             // [2][G][32][ldk]
  __nv_bfloat16* v_s = k_s + 2 * G * TM_KT * ldk;                     // [2][G][32][ldk]
  float* r_s = reinterpret_cast<float*>(v_s + 2 * G * TM_KT * ldk);   // [H][4][32 lanes][4]: a lane's own accumulators
  float* t_s = r_s + H * TM_BQ * TM_KT;                               // [H][H]
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.y;
  const int t0 = p.seq_start[seq], n_new = p.seq_start[seq + 1] - t0;
  const bool split = p.n_split > 1;
  const int q0 = split ? 0 : ((int)gridDim.x - 1 - (int)blockIdx.x) * TM_BQ;      // (the last tiles see the most keys: first)
  if (q0 >= n_new) return;
  const int nq = min(TM_BQ, n_new - q0);
  const int past = p.past_len[seq];
  const int tid = threadIdx.x, n_threads = blockDim.x, lane = tid & 31, head = tid >> 5, g = lane >> 2, qd = lane & 3;
  const int kv_head = head / (H / G);
  const int chunks = D / 8;
  constexpr int dchunks = dp / 8;
  for (int i = tid; i < TM_BQ * H * dchunks; i += n_threads) {
    const int r = i / (H * dchunks), rest = i - r * H * dchunks, h = rest / dchunks, c = rest - h * dchunks;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (r < nq && c < chunks) val = *reinterpret_cast<const uint4*>(p.q + (long long)(t0 + q0 + r) * p.q_row + h * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + r * ldq + h * dp + c * 8) = val;
  }
  for (int i = tid; i < H * H; i += n_threads) t_s[i] = (p.talk ? p.talk[i] : (i / H == i % H ? 1.f : 0.f)) * LOG2E;
  // channels past head_dim of the key and value tiles, which no copy writes
  if (chunks < dchunks)
    for (int i = tid; i < 2 * 2 * G * TM_KT * (dchunks - chunks); i += n_threads) {
      const int row = i / (dchunks - chunks), c = chunks + i - row * (dchunks - chunks);
      *reinterpret_cast<uint4*>(k_s + row * ldk + c * 8) = make_uint4(0u, 0u, 0u, 0u);      // (v_s follows k_s: rows of both)
    }
  const int pos_first = past + q0, pos_last = past + q0 + nq - 1;
  const int k_hi = pos_last + 1;                                               // exclusive
  const int k_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
  const int tile_step = split ? p.n_split : 1;
  const int tile_lo = k_lo / TM_KT + (split ? (int)blockIdx.x : 0), tile_hi = (k_hi + TM_KT - 1) / TM_KT;
  if (tile_lo >= tile_hi) return;               // (a short sequence has fewer tiles than the step has blocks for it)
  // a tile's 32 positions lie in one page when a page holds a multiple of 32
  const bool one_page = p.kv.table != nullptr && p.kv.page_size % TM_KT == 0;
  auto load_tile = [&](int tile, int buf) {
    __nv_bfloat16* kd = k_s + buf * G * TM_KT * ldk;
    __nv_bfloat16* vd = v_s + buf * G * TM_KT * ldk;
    long long tile_at = 0, head_step = D, row_step = D;      // elements: the tile's first row of key head 0, between heads, rows
    if (one_page) {
      const int lp = tile * TM_KT / p.kv.page_size;
      const int page = p.kv.table[(long long)seq * p.kv.table_stride + (lp % p.kv.table_len)];
      tile_at = ((long long)page * G * p.kv.page_size + (tile * TM_KT - lp * p.kv.page_size)) * D;
      head_step = (long long)p.kv.page_size * D;
    } else if (!p.kv.table) {
      tile_at = ((long long)p.kv.seq_start[seq] + tile * TM_KT) * p.kv.row_stride;
      row_step = p.kv.row_stride;
    }
    for (int i = tid; i < G * TM_KT * dchunks; i += n_threads) {
      const int c = i % dchunks, r = (i / dchunks) % TM_KT, gk = i / (dchunks * TM_KT);
      if (c >= chunks) continue;
      const int kp = tile * TM_KT + r;
      const bool ok = kp >= k_lo && kp < k_hi;
      const unsigned off = (unsigned)((gk * TM_KT + r) * ldk + c * 8);
      const __nv_bfloat16 *ksrc, *vsrc;
      if (one_page || !p.kv.table) {
        const long long at = ok ? tile_at + gk * head_step + r * row_step + c * 8 : 0;
        ksrc = reinterpret_cast<const __nv_bfloat16*>(p.kv.k) + at;
        vsrc = reinterpret_cast<const __nv_bfloat16*>(p.kv.v) + at;
      } else {
        ksrc = kv_row<__nv_bfloat16>(p.kv.k, p.kv, seq, gk, G, D, ok ? kp : k_lo) + c * 8;
        vsrc = kv_row<__nv_bfloat16>(p.kv.v, p.kv, seq, gk, G, D, ok ? kp : k_lo) + c * 8;
      }
      tm_cp_async16(ds_smem(kd + off), ksrc, ok ? 16 : 0);
      tm_cp_async16(ds_smem(vd + off), vsrc, ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  load_tile(tile_lo, 0);
  const float my_scale = p.scale * (p.temp ? p.temp[head] : 1.f);
  const float my_slope = p.slope ? p.slope[head] : 0.f;
  const float two_inv_cap = p.cap > 0.f ? 2.f / p.cap : 0.f;
  const int qpos0 = past + q0 + g;                       // the lane's rows: this position and the one 8 further
  const int seen_span = p.window > 0 ? p.window : 0x7fffffff;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float acc[2 * NP][4];
#pragma unroll
  for (int j = 0; j < 2 * NP; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
  const unsigned q_addr = ds_smem(q_s + (lane & 15) * ldq + head * dp + (lane >> 4) * 8);
  const int mi = lane >> 3, lr = lane & 7;
  // what this lane names for ldmatrix inside a tile of its key head: keys as the 8-column operand (rows = keys), values
  // transposed (rows = keys, 8 channels a row)
  const unsigned k_lane = (unsigned)(((kv_head * TM_KT + (mi >> 1) * 8 + lr) * ldk + (mi & 1) * 8) * 2);
  const unsigned v_lane = (unsigned)(((kv_head * TM_KT + (mi & 1) * 8 + lr) * ldk + (mi >> 1) * 8) * 2);
  float* r_mine = r_s + head * (NT * 128);

  for (int tile = tile_lo, buf = 0; tile < tile_hi; tile += tile_step, buf ^= 1) {
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    if (tile + tile_step < tile_hi) load_tile(tile + tile_step, buf ^ 1);
    const unsigned kt = ds_smem(k_s + buf * G * TM_KT * ldk), vt = ds_smem(v_s + buf * G * TM_KT * ldk);
    const int key0 = tile * TM_KT;
    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < NP; ++ks) {
      unsigned a[4];
      ds_ldmatrix_x4(a, q_addr + ks * 32);
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {
        unsigned b[4];
        ds_ldmatrix_x4(b, kt + k_lane + (unsigned)(n2 * 16 * ldk * 2) + ks * 32);
        ds_mma(s[2 * n2], a[0], a[1], a[2], a[3], b[0], b[1]);
        ds_mma(s[2 * n2 + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
      }
    }
    // this head's raw scores: scale and temperature, the cap, the distance's bias.  rel0: how far the lane's first key
    // lies behind its first row; element (n, e) lies 8 (e >> 1) - 8 n - (e & 1) further
    const int rel0 = qpos0 - key0 - qd * 2;
    const float bias0 = my_slope * (float)rel0;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x = s[n][e] * my_scale;
        if (p.cap > 0.f) x = p.cap * (1.f - __fdividef(2.f, __expf(x * two_inv_cap) + 1.f));
        s[n][e] = x - fmaf(my_slope, (float)(8 * (e >> 1) - 8 * n - (e & 1)), bias0);
      }
      *reinterpret_cast<float4*>(r_mine + (n * 32 + lane) * 4) = make_float4(s[n][0], s[n][1], s[n][2], s[n][3]);
    }
    __syncthreads();
    // the heads' planes summed with this head's row of `talk` (times log2 e: the softmax works in base 2)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
    for (int h2 = 0; h2 < H; ++h2) {
      const float w = t_s[head * H + h2];
      const float* src = r_s + h2 * (NT * 128) + lane * 4;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const float4 x = *reinterpret_cast<const float4*>(src + n * 128);
        s[n][0] = fmaf(w, x.x, s[n][0]);
        s[n][1] = fmaf(w, x.y, s[n][1]);
        s[n][2] = fmaf(w, x.z, s[n][2]);
        s[n][3] = fmaf(w, x.w, s[n][3]);
      }
    }
    // every key of the tile before every row of the block and inside its window: nothing to hide
    const bool full = key0 + TM_KT - 1 <= pos_first && pos_first + TM_BQ - 1 - key0 < seen_span;
    if (!full) {
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int rel = rel0 + 8 * (e >> 1) - 8 * n - (e & 1);
          if ((unsigned)rel >= (unsigned)seen_span) s[n][e] = -INFINITY;
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
    float corr[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      mx[u] = fmaxf(mx[u], __shfl_xor_sync(0xffffffffu, mx[u], 1));
      mx[u] = fmaxf(mx[u], __shfl_xor_sync(0xffffffffu, mx[u], 2));
      const float m_new = fmaxf(m_run[u], mx[u]);
      corr[u] = m_new == -INFINITY ? 1.f : ds_exp2(m_run[u] - m_new);
      m_run[u] = m_new;
    }
    // (a row that has seen no key yet keeps the maximum -inf; its weights are 2^(-inf - 0) = 0)
    const float m_use[2] = {m_run[0] == -INFINITY ? 0.f : m_run[0], m_run[1] == -INFINITY ? 0.f : m_run[1]};
    float psum[2] = {0.f, 0.f};
    unsigned p_hi[NT][2], p_lo[NT][2];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      float w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        w[e] = ds_exp2(s[n][e] - m_use[e >> 1]);
        psum[e >> 1] += w[e];
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const __nv_bfloat162 hi = __floats2bfloat162_rn(w[2 * u], w[2 * u + 1]);
        const float2 back = __bfloat1622float2(hi);
        p_hi[n][u] = *reinterpret_cast<const unsigned*>(&hi);
        p_lo[n][u] = ds_pack(w[2 * u] - back.x, w[2 * u + 1] - back.y);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) l_run[u] = l_run[u] * corr[u] + psum[u];
#pragma unroll
    for (int j = 0; j < 2 * NP; ++j) {
      acc[j][0] *= corr[0];
      acc[j][1] *= corr[0];
      acc[j][2] *= corr[1];
      acc[j][3] *= corr[1];
    }
#pragma unroll
    for (int kb = 0; kb < NT / 2; ++kb) {
#pragma unroll
      for (int jp = 0; jp < NP; ++jp) {
        unsigned b[4];
        ds_ldmatrix_x4_trans(b, vt + v_lane + (unsigned)(kb * 16 * ldk * 2) + jp * 32);
        ds_mma(acc[2 * jp], p_hi[2 * kb][0], p_hi[2 * kb][1], p_hi[2 * kb + 1][0], p_hi[2 * kb + 1][1], b[0], b[1]);
        ds_mma(acc[2 * jp], p_lo[2 * kb][0], p_lo[2 * kb][1], p_lo[2 * kb + 1][0], p_lo[2 * kb + 1][1], b[0], b[1]);
        ds_mma(acc[2 * jp + 1], p_hi[2 * kb][0], p_hi[2 * kb][1], p_hi[2 * kb + 1][0], p_hi[2 * kb + 1][1], b[2], b[3]);
        ds_mma(acc[2 * jp + 1], p_lo[2 * kb][0], p_lo[2 * kb][1], p_lo[2 * kb + 1][0], p_lo[2 * kb + 1][1], b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    float l = l_run[u];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int r = g + 8 * u;
    if (r >= nq) continue;
    if (split) {
      float* part = p.parts + ((((long long)seq * p.n_split + blockIdx.x) * H + head) * p.max_new + r) * (D + 2);
#pragma unroll
      for (int j = 0; j < 2 * NP; ++j) {
        const int c = j * 8 + qd * 2;
        if (c < D) *reinterpret_cast<float2*>(part + c) = make_float2(acc[j][2 * u], acc[j][2 * u + 1]);
      }
      if (qd == 0) *reinterpret_cast<float2*>(part + D) = make_float2(m_run[u], l);
      continue;
    }
    const float inv = l > 0.f ? p.out_scale / l : 0.f;
    const long long t = t0 + q0 + r;
#pragma unroll
    for (int j = 0; j < 2 * NP; ++j) {
      const int c = j * 8 + qd * 2;
      if (c >= D) continue;
      float y0 = acc[j][2 * u] * inv, y1 = acc[j][2 * u + 1] * inv;
      if (p.gate) {
        const float2 gt = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p.gate + t * p.gate_row + head * D + c));
        y0 *= 1.f / (1.f + expf(-gt.x));
        y1 *= 1.f / (1.f + expf(-gt.y));
      }
      *reinterpret_cast<__nv_bfloat162*>(p.out + t * p.out_row + head * D + c) = __floats2bfloat162_rn(y0, y1);
    }
  }
}

// Joins what the blocks of a sequence left in `parts`: a block a (row, sequence), a thread a pair of channels.
__global__ void __launch_bounds__(128) talking_attention_join_kernel(TalkingArgs p) {
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.y, r = blockIdx.x;
  const int t0 = p.seq_start[seq], n_new = p.seq_start[seq + 1] - t0;
  if (r >= n_new) return;
  const int H = p.n_heads, D = p.head_dim;
  const int past = p.past_len[seq];
  const int k_hi = past + min(TM_BQ, n_new);
  const int k_lo = p.window > 0 ? max(0, past - p.window + 1) : 0;
  const int n_parts = min(p.n_split, (k_hi + TM_KT - 1) / TM_KT - k_lo / TM_KT);
  const long long t = t0 + r;
  for (int i = threadIdx.x; i < H * D / 2; i += blockDim.x) {
    const int head = i / (D / 2), c = (i - head * (D / 2)) * 2;
    const float* first = p.parts + (((long long)seq * p.n_split * H + head) * p.max_new + r) * (D + 2);
    const long long step = (long long)H * p.max_new * (D + 2);
    float m = -INFINITY;
    for (int b = 0; b < n_parts; ++b) m = fmaxf(m, first[b * step + D]);
    float l = 0.f, y0 = 0.f, y1 = 0.f;
    for (int b = 0; b < n_parts; ++b) {
      const float* part = first + b * step;
      const float w = part[D] == -INFINITY ? 0.f : ds_exp2(part[D] - m);
      const float2 a = *reinterpret_cast<const float2*>(part + c);
      l = fmaf(w, part[D + 1], l);
      y0 = fmaf(w, a.x, y0);
      y1 = fmaf(w, a.y, y1);
    }
    const float inv = l > 0.f ? p.out_scale / l : 0.f;
    y0 *= inv;
    y1 *= inv;
    if (p.gate) {
      const float2 gt = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p.gate + t * p.gate_row + head * D + c));
      y0 *= 1.f / (1.f + expf(-gt.x));
      y1 *= 1.f / (1.f + expf(-gt.y));
    }
    *reinterpret_cast<__nv_bfloat162*>(p.out + t * p.out_row + head * D + c) = __floats2bfloat162_rn(y0, y1);
  }
}

template <int NP, int WB>
static int tm_launch(const TalkingArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
  auto kern = talking_attention_mma_kernel<NP, WB>;
  if (smem > 48 * 1024)
    BT_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess,
             "talking_attention: cannot reserve %zu bytes of shared memory", smem);
  BT_PDL_OK("talking_attention_mma", launch_pdl(kern, grid, dim3(32 * a.n_heads), smem, stream, 1, a));
  return 0;
}

template <int NP>
static int tm_launch_heads(const TalkingArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
  if (a.n_heads <= 8) return tm_launch<NP, 8>(a, grid, smem, stream);
  if (a.n_heads <= 16) return tm_launch<NP, 16>(a, grid, smem, stream);
  return tm_launch<NP, 32>(a, grid, smem, stream);
}

// Whether the tensor-core form takes these rows: heads of a multiple of 8 channels up to 128, 16-byte aligned rows,
// and tiles that fit shared memory.
static bool tm_takes(const TalkingArgs& a) {
  if (a.head_dim % 8 || a.head_dim > 128) return false;
  auto aligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
  if (!aligned(a.q) || !aligned(a.kv.k) || !aligned(a.kv.v) || !aligned(a.out) || (a.gate && !aligned(a.gate))) return false;
  if (a.q_row % 8 || a.out_row % 8 || (a.gate && a.gate_row % 8) || (!a.kv.table && a.kv.row_stride % 8)) return false;
  return tm_smem(a.n_heads, a.n_kv_heads, (a.head_dim + 15) & ~15) <= 200 * 1024;
}

static int talking_mma_launch(const TalkingArgs& a, int n_seqs, int max_new, cudaStream_t stream) {
  const int np = (a.head_dim + 15) / 16;
  const dim3 grid(a.n_split > 1 ? a.n_split : (max_new + TM_BQ - 1) / TM_BQ, n_seqs);
  const size_t smem = tm_smem(a.n_heads, a.n_kv_heads, np * 16);
  switch (np) {
    case 1: return tm_launch_heads<1>(a, grid, smem, stream);
    case 2: return tm_launch_heads<2>(a, grid, smem, stream);
    case 3: return tm_launch_heads<3>(a, grid, smem, stream);
    case 4: return tm_launch_heads<4>(a, grid, smem, stream);
    case 5: return tm_launch_heads<5>(a, grid, smem, stream);
    case 6: return tm_launch_heads<6>(a, grid, smem, stream);
    case 7: return tm_launch_heads<7>(a, grid, smem, stream);
    case 8: return tm_launch_heads<8>(a, grid, smem, stream);
  }
  return fail("talking_attention: head_dim %d has no tensor-core form", a.head_dim);
}

// Runs the tensor-core form if it takes these rows (bfloat16); *taken says whether it did.
// n_split > 1 (only with max_new <= 16): the keys of every sequence are shared by n_split blocks that meet in `parts`
// (n_seqs * n_split * n_heads * max_new * (head_dim + 2) floats).
int talking_attention_mma(const void* q, long long q_row_stride, const KvView& view, const void* gate,
                          long long gate_row_stride, void* out, long long out_row_stride, const int* seq_start,
                          const int* past_len, const float* temp, const float* slope, const float* talk, int n_seqs,
                          int max_new, int n_heads, int n_kv_heads, int head_dim, float scale, float cap, int window,
                          float out_scale, int n_split, float* parts, cudaStream_t stream, bool* taken) {
  if (n_split > 1 && (max_new > TM_BQ || parts == nullptr)) n_split = 1;
  TalkingArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)gate, (__nv_bfloat16*)out, q_row_stride, gate_row_stride,
                out_row_stride, view, seq_start, past_len, temp, slope, talk, n_heads, n_kv_heads, head_dim, scale, cap,
                out_scale, window, n_split, max_new, parts};
  *taken = tm_takes(a);
  if (!*taken) return 0;
  const int rc = talking_mma_launch(a, n_seqs, max_new, stream);
  if (rc || n_split <= 1) return rc;
  BT_PDL_OK("talking_attention_join", launch_pdl(talking_attention_join_kernel, dim3(max_new, n_seqs), dim3(128), 0, stream,
                                                 1, a));
  return 0;
}

}  // namespace bt
