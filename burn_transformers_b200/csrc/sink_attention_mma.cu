// Causal multi-head attention of fresh prompts on tensor cores (bfloat16), with an optional per-head sink in the
// softmax denominator and an optional sigmoid gate on the result: the plain form of the latent attention for steps in
// which every sequence starts at position 0, so that keys and values are the step's own rows (up-projected per head by
// the caller).  It does dq + dv multiply-adds a key and head where the form that carries the query into the latent
// space does 2 rank + rot.
//
// A block is 64 query tokens of one head of one sequence, four warps of 16 rows; key and value tiles of 64 tokens come
// through two cp.async buffers; scores and value mix are mma.sync products, the weights pass from the scores'
// accumulators to the value product's operand inside registers; softmax, sink and accumulators are 32-bit.
// (Tried and not kept: eight warps as two groups that take the key tiles in turn and join at the end.  It halves the
// chain of tiles the last rows of a prompt walk, but a block then holds twice the buffers and registers: 72 against 77 us
// for 2 x 1,024 tokens of 12 heads, 113 against 97 us for 16 heads, where the blocks no longer fit the GPU at once.)
#include "decode_mma.cuh"

namespace bt {

constexpr int SA_BM = 64, SA_KT = 64, SA_PAD = 8;
constexpr int SA_NT = SA_KT / 8;      // 8-key score tiles per key tile

__device__ __forceinline__ void sa_ldmatrix_x2(unsigned (&r)[2], unsigned smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_addr));
}
__device__ __forceinline__ void sa_cp_async16(unsigned dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

struct SinkAttentionArgs {
  const __nv_bfloat16 *q, *k, *v, *gate;
  __nv_bfloat16* out;
  long long q_row, k_row, v_row, gate_row, out_row;     // elements between tokens
  int q_head, k_head, v_head, gate_head, out_head;      // elements between heads
  const int* seq_start;
  const float* sink;
  int dq, dv;
  float scale;
  int window;      // > 0: a row sees the last `window` positions up to its own
  int keep_first;  // with a window: positions below this stay visible to every later row
  int kv_group;    // query heads that share a key and value head (1: every head has its own)
  const float* bias;   // SIGMOID: a number per head added to the scaled score
};

// VCT: the most value channels (a multiple of 16).  SIGMOID: the weight of a visible key is sigmoid(score * scale + bias[head])
// and nothing is normalised over the keys (no running maximum, no denominator, no sink).
template <int VCT, bool SIGMOID>
__global__ void __launch_bounds__(128) sink_attention_mma_kernel(SinkAttentionArgs p) {
  extern __shared__ __align__(16) unsigned char sa_smem[];
  constexpr int NP = VCT / 16;
  constexpr float LOG2E = 1.4426950408889634f;
  const int dqp = (p.dq + 15) & ~15, ldq = dqp + SA_PAD;
  const int dvp = (p.dv + 15) & ~15, ldv = dvp + SA_PAD;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(sa_smem);   // [64][ldq]
  __nv_bfloat16* k_s = q_s + SA_BM * ldq;                           // [2][SA_KT][ldq]
  __nv_bfloat16* v_s = k_s + 2 * SA_KT * ldq;                       // [2][SA_KT][ldv]
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int tile = gridDim.x - 1 - blockIdx.x;                      // the longest tiles start first
  const int first = p.seq_start[seq], n_new = p.seq_start[seq + 1] - first;
  const int t0 = tile * SA_BM;
  if (t0 >= n_new) return;
  const int n_valid = min(SA_BM, n_new - t0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, qd = lane & 3;
  const bool active = warp * 16 < n_valid;
  const int q_chunks = dqp / 8;
  for (int i = tid; i < SA_BM * q_chunks; i += 128) {
    const int r = i / q_chunks, c = i - r * q_chunks;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (r < n_valid && c * 8 < p.dq)
      val = *reinterpret_cast<const uint4*>(p.q + (long long)(first + t0 + r) * p.q_row + (long long)head * p.q_head + c * 8);
    *reinterpret_cast<uint4*>(q_s + r * ldq + c * 8) = val;
  }
  // channels past dq / dv of the key and value tiles, which no copy writes
  if (dqp > p.dq)
    for (int i = tid; i < 2 * SA_KT; i += 128) *reinterpret_cast<uint4*>(k_s + i * ldq + p.dq) = make_uint4(0u, 0u, 0u, 0u);
  if (dvp > p.dv)
    for (int i = tid; i < 2 * SA_KT; i += 128) *reinterpret_cast<uint4*>(v_s + i * ldv + p.dv) = make_uint4(0u, 0u, 0u, 0u);
  const int last = t0 + n_valid - 1;                 // the last key any row of the block sees
  const int n_tiles = last / SA_KT + 1;
  const int kq = p.dq / 8, kv = p.dv / 8;
  const int kv_head = head / p.kv_group;
  auto load_tile = [&](int kt, int buf) {
    const int j0 = kt * SA_KT;
    __nv_bfloat16* kd = k_s + buf * SA_KT * ldq;
    __nv_bfloat16* vd = v_s + buf * SA_KT * ldv;
    for (int i = tid; i < SA_KT * (kq + kv); i += 128) {
      const int kk = i / (kq + kv), c = i - kk * (kq + kv);
      const int j = j0 + kk;
      const bool ok = j <= last;
      const long long tok = first + (ok ? j : 0);
      if (c < kq)
        sa_cp_async16(ds_smem(kd + kk * ldq + c * 8), p.k + tok * p.k_row + (long long)kv_head * p.k_head + c * 8, ok ? 16 : 0);
      else
        sa_cp_async16(ds_smem(vd + kk * ldv + (c - kq) * 8), p.v + tok * p.v_row + (long long)kv_head * p.v_head + (c - kq) * 8,
                      ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  // tiles before kt_first lie outside every row's window; those that hold kept first positions are walked all the same
  const int kt_first = p.window > 0 ? max(0, t0 - p.window + 1) / SA_KT : 0;
  const int kept_tiles = p.window > 0 ? (min(p.keep_first, last + 1) + SA_KT - 1) / SA_KT : 0;
  auto next_tile = [&](int kt) {
    const int n = kt + 1;
    return (n >= kept_tiles && n < kt_first) ? kt_first : n;
  };
  const int kt_begin = kept_tiles > 0 ? 0 : kt_first;
  load_tile(kt_begin, 0);
  float m_run[2], l_run[2];
  const bool has_sink = !SIGMOID && p.sink != nullptr;
  const float bias_log2 = SIGMOID && p.bias != nullptr ? p.bias[head] * LOG2E : 0.f;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    m_run[e] = has_sink ? p.sink[head] * LOG2E : -INFINITY;
    l_run[e] = has_sink ? 1.f : 0.f;
  }
  float acc[2 * NP][4];
#pragma unroll
  for (int j = 0; j < 2 * NP; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
  const float scale_log2 = p.scale * LOG2E;
  const int row0 = t0 + warp * 16 + g;               // this lane's rows: row0 and row0 + 8 (positions inside the sequence)
  const unsigned q_addr = ds_smem(q_s + (warp * 16 + (lane & 15)) * ldq + (lane >> 4) * 8);
  const int blk = lane >> 3;
  for (int kt = kt_begin, round = 0; kt < n_tiles; kt = next_tile(kt), ++round) {
    const int buf = round & 1;
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    if (next_tile(kt) < n_tiles) load_tile(next_tile(kt), buf ^ 1);
    const int j0 = kt * SA_KT;
    if (!active || j0 > t0 + warp * 16 + 15) continue;      // (no row of this warp sees the tile)
    const __nv_bfloat16* ktile = k_s + buf * SA_KT * ldq;
    const __nv_bfloat16* vtile = v_s + buf * SA_KT * ldv;
    float s[SA_NT][4];
#pragma unroll
    for (int n = 0; n < SA_NT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
    const unsigned k_addr = ds_smem(ktile + (lane & 7) * ldq + ((lane >> 3) & 1) * 8);
#pragma unroll 2
    for (int ks = 0; ks < dqp / 16; ++ks) {
      unsigned a[4];
      ds_ldmatrix_x4(a, q_addr + ks * 32);
#pragma unroll
      for (int n = 0; n < SA_NT; ++n) {
        unsigned b[2];
        sa_ldmatrix_x2(b, k_addr + (unsigned)(n * 8 * ldq * 2) + ks * 32);
        ds_mma(s[n], a[0], a[1], a[2], a[3], b[0], b[1]);
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < SA_NT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + n * 8 + qd * 2 + (e & 1);
        const int rr = e >> 1;
        const int row = row0 + 8 * rr;
        const bool seen = row < n_new && j <= row && (p.window <= 0 || row - j < p.window || j < p.keep_first);
        const float val = seen ? s[n][e] * scale_log2 : -INFINITY;
        s[n][e] = val;
        mx[rr] = fmaxf(mx[rr], val);
      }
    unsigned pa[SA_KT / 16][4];                               // the weights as the value product's first operand, per 16 keys
    if (SIGMOID) {
#pragma unroll
      for (int n = 0; n < SA_NT; ++n) {
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) pv[e] = s[n][e] == -INFINITY ? 0.f : 1.f / (1.f + ds_exp2(-(s[n][e] + bias_log2)));
        pa[n >> 1][(n & 1) * 2] = ds_pack(pv[0], pv[1]);
        pa[n >> 1][(n & 1) * 2 + 1] = ds_pack(pv[2], pv[3]);
      }
    } else {
    float corr[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
      const float m_new = fmaxf(m_run[rr], mx[rr]);
      corr[rr] = m_new == -INFINITY ? 1.f : ds_exp2(m_run[rr] - m_new);
      m_run[rr] = m_new;
    }
    float ps[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < SA_NT; ++n) {
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pv[e] = s[n][e] == -INFINITY ? 0.f : ds_exp2(s[n][e] - m_run[e >> 1]);
        ps[e >> 1] += pv[e];
      }
      pa[n >> 1][(n & 1) * 2] = ds_pack(pv[0], pv[1]);
      pa[n >> 1][(n & 1) * 2 + 1] = ds_pack(pv[2], pv[3]);
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      ps[rr] += __shfl_xor_sync(0xffffffffu, ps[rr], 1);
      ps[rr] += __shfl_xor_sync(0xffffffffu, ps[rr], 2);
      l_run[rr] = l_run[rr] * corr[rr] + ps[rr];
    }
#pragma unroll
    for (int j = 0; j < 2 * NP; ++j) {
      acc[j][0] *= corr[0];
      acc[j][1] *= corr[0];
      acc[j][2] *= corr[1];
      acc[j][3] *= corr[1];
    }
    }
    const unsigned v_addr = ds_smem(vtile + ((blk & 1) * 8 + (lane & 7)) * ldv + (blk >> 1) * 8);
#pragma unroll
    for (int k2 = 0; k2 < SA_KT / 16; ++k2) {
#pragma unroll
      for (int np = 0; np < NP; ++np) {
        if (np * 16 < dvp) {
          unsigned b[4];
          ds_ldmatrix_x4_trans(b, v_addr + (unsigned)(k2 * 16 * ldv * 2) + np * 32);
          ds_mma(acc[2 * np], pa[k2][0], pa[k2][1], pa[k2][2], pa[k2][3], b[0], b[1]);
          ds_mma(acc[2 * np + 1], pa[k2][0], pa[k2][1], pa[k2][2], pa[k2][3], b[2], b[3]);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  if (!active) return;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int row = row0 + 8 * rr;
    if (row >= n_new) continue;
    const float inv = SIGMOID ? 1.f : (l_run[rr] > 0.f ? 1.f / l_run[rr] : 0.f);
    const long long tok = first + row;
    __nv_bfloat16* dst = p.out + tok * p.out_row + (long long)head * p.out_head;
    const __nv_bfloat16* gt = p.gate ? p.gate + tok * p.gate_row + (long long)head * p.gate_head : nullptr;
#pragma unroll
    for (int j = 0; j < 2 * NP; ++j) {
      const int c = j * 8 + qd * 2;
      if (c >= p.dv) continue;
      float v0 = acc[j][2 * rr] * inv, v1 = acc[j][2 * rr + 1] * inv;
      if (gt) {
        const float2 gv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gt + c));
        v0 *= 1.f / (1.f + expf(-gv.x));
        v1 *= 1.f / (1.f + expf(-gv.y));
      }
      *reinterpret_cast<unsigned*>(dst + c) = ds_pack(v0, v1);
    }
  }
}

}  // namespace bt

// 1 if the operands lie so that the kernel takes them: whole 16-byte pieces per head and row, at most 128 value channels.
extern "C" int bt_sink_attention_supports(int dq, int dv, long long q_row, int q_head, long long k_row, int k_head,
                                          long long v_row, int v_head, long long gate_row, int gate_head,
                                          long long out_row, int out_head) {
  return dq > 0 && dv > 0 && dq % 8 == 0 && dv % 8 == 0 && dv <= 128 && dq <= 512 && q_row % 8 == 0 && q_head % 8 == 0 &&
         k_row % 8 == 0 && k_head % 8 == 0 && v_row % 8 == 0 && v_head % 8 == 0 && gate_row % 2 == 0 && gate_head % 2 == 0 &&
         out_row % 2 == 0 && out_head % 2 == 0;
}

extern "C" int bt_sink_attention(const void* q, long long q_row, int q_head, const void* k, long long k_row, int k_head,
                                 const void* v, long long v_row, int v_head, const void* gate, long long gate_row,
                                 int gate_head, void* out, long long out_row, int out_head, const int* seq_start,
                                 const float* sink, int n_seqs, int max_new, int n_heads, int dq, int dv, float scale,
                                 int window, int keep_first, int kv_group, int sigmoid, const float* bias,
                                 cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(bt_sink_attention_supports(dq, dv, q_row, q_head, k_row, k_head, v_row, v_head, gate_row, gate_head, out_row,
                                      out_head),
           "sink_attention: sizes or strides the kernel does not take (dq=%d dv=%d)", dq, dv);
  auto at = [](const void* ptr, int bytes) { return ((unsigned long long)ptr % bytes) == 0; };
  BT_CHECK(at(q, 16) && at(k, 16) && at(v, 16) && at(out, 4) && (gate == nullptr || at(gate, 4)),
           "sink_attention: operands must lie on 16-byte boundaries");
  BT_CHECK(n_heads > 0 && n_heads <= 65535 && n_seqs <= 65535 && kv_group > 0 && n_heads % kv_group == 0 && window >= 0 &&
               keep_first >= 0,
           "sink_attention: bad sizes heads=%d seqs=%d heads a key head=%d", n_heads, n_seqs, kv_group);
  if (n_seqs == 0 || max_new == 0) return 0;
  SinkAttentionArgs p;
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
  p.gate = (const __nv_bfloat16*)gate; p.out = (__nv_bfloat16*)out;
  p.q_row = q_row; p.k_row = k_row; p.v_row = v_row; p.gate_row = gate_row; p.out_row = out_row;
  p.q_head = q_head; p.k_head = k_head; p.v_head = v_head; p.gate_head = gate_head; p.out_head = out_head;
  p.seq_start = seq_start; p.sink = sink; p.dq = dq; p.dv = dv; p.scale = scale; p.window = window;
  p.keep_first = keep_first; p.kv_group = kv_group; p.bias = bias;
  const int dqp = (dq + 15) & ~15, dvp = (dv + 15) & ~15;
  const size_t smem = (size_t)(SA_BM + 2 * SA_KT) * (dqp + SA_PAD) * 2 + (size_t)2 * SA_KT * (dvp + SA_PAD) * 2;
  const dim3 grid((max_new + SA_BM - 1) / SA_BM, n_heads, n_seqs), block(128);
#define BT_SA(VCT)                                                                                                \
  do {                                                                                                            \
    if (sigmoid) BT_SA_KIND(VCT, true); else BT_SA_KIND(VCT, false);                                              \
  } while (0)
#define BT_SA_KIND(VCT, SIGMOID)                                                                                  \
  do {                                                                                                            \
    auto kernel = sink_attention_mma_kernel<VCT, SIGMOID>;                                                        \
    static size_t reserved = 0;                                                                                   \
    if (smem > 48 * 1024 && smem > reserved) {                                                                    \
      BT_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess, \
               "sink_attention: cannot reserve %zu bytes of shared memory", smem);                                \
      reserved = smem;                                                                                            \
    }                                                                                                             \
    BT_PDL_OK("sink_attention", launch_pdl(kernel, grid, block, smem, stream, 1, p));                             \
  } while (0)
  if (dvp <= 32) BT_SA(32);
  else if (dvp <= 64) BT_SA(64);
  else BT_SA(128);
#undef BT_SA
#undef BT_SA_KIND
  return 0;
}
