// Attention over a latent cache on tensor cores (bfloat16): the same computation as latent_attention_kernel in
// latent_attention.cu, with the scores and the value mix as mma.sync products.
//
// A block holds 64 rows, (token, head) pairs of one sequence, which all read the same key tiles of 32 cached rows.
// Warps form 4 row groups of 16 rows; VW warps share a row group.  Per tile a warp computes the scores of its rows
// against its 32 / VW keys over all rank + rot channels; the warps of a group exchange row maxima and sums through shared
// memory and leave their weights there as bfloat16; then every warp multiplies the group's 16 x 32 weights with ITS
// rank / VW channels of the tile's rows (values are the first `rank` channels of the key rows).  So no score is
// computed twice and a warp's accumulator stays at 16 x 128 numbers at most.  Key tiles arrive by cp.async into two
// buffers, the next tile's copy running under the current tile's products.  Scores, maxima, sums and accumulators are
// 32-bit; the weights are rounded to bfloat16 as the operand of the value product.
#include "decode_mma.cuh"

namespace bt {

constexpr int LM_BM = 64;
constexpr int LM_KT = 32;
constexpr int LM_PAD = 8;                 // elements: rows of shared memory lie an odd number of 16-byte pieces apart
constexpr int LM_PLD = LM_KT + LM_PAD;    // row length of the weights' tile

__device__ __forceinline__ void lm_ldmatrix_x2(unsigned (&r)[2], unsigned smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_addr));
}
__device__ __forceinline__ void lm_cp_async16(unsigned dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void lm_cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void lm_cp_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// VW: warps per row group; VCT: the most value channels a warp owns (its accumulator's size)
template <int VW, int VCT>
__global__ void __launch_bounds__(128 * VW)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, long long q_row_stride,
                            const __nv_bfloat16* __restrict__ pool, const int* __restrict__ table, int table_stride,
                            int table_len, int page_size, const int* __restrict__ seq_start,
                            const int* __restrict__ past_len, const float* __restrict__ sink,
                            __nv_bfloat16* __restrict__ out, long long out_row_stride, float* __restrict__ part,
                            int n_heads, int hb, int tq, int head_tiles, int rank, int rot, float scale, int n_splits,
                            int window) {
  extern __shared__ __align__(16) unsigned char lm_smem[];
  constexpr int NT = LM_KT / VW / 8;        // 8-key score tiles per warp
  constexpr int NP = VCT / 16;              // pairs of 8-channel value tiles per warp
  constexpr float LOG2E = 1.4426950408889634f;
  const int dk = rank + rot, dkp = (dk + 15) & ~15, ld = dkp + LM_PAD;
  const int vc = rank / VW;                 // value channels per warp
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(lm_smem);   // [64][ld]
  __nv_bfloat16* k_s = q_s + LM_BM * ld;                            // [2][32][ld]
  __nv_bfloat16* p_s = k_s + 2 * LM_KT * ld;                        // [4][16][LM_PLD]
  float* red_max = reinterpret_cast<float*>(p_s + 4 * 16 * LM_PLD); // [4][VW][16]
  float* red_sum = red_max + 4 * VW * 16;                           // [4][VW][16]
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.z, split = blockIdx.y;
  // (the last tokens of a prompt see the most keys: their tiles come first, so that the longest blocks start first)
  const int token_tiles = gridDim.x / head_tiles;
  const int token_tile = token_tiles - 1 - blockIdx.x / head_tiles, head_tile = blockIdx.x % head_tiles;
  const int first = seq_start[seq], n_new = seq_start[seq + 1] - first, past = past_len[seq];
  const int t0 = token_tile * tq;
  if (t0 >= n_new) return;
  const int h0 = head_tile * hb;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp / VW, vw = warp - rg * VW;
  const int n_valid = head_tiles == 1 ? min(tq, n_new - t0) * hb : min(hb, n_heads - h0);   // valid rows are the first ones
  const bool active = rg * 16 < n_valid;
  const int chunks = dkp / 8;               // 16-byte pieces per row
  // the block's queries; rows past the valid ones and channels past rank + rot are zeros
  for (int i = tid; i < LM_BM * chunks; i += blockDim.x) {
    const int r = i / chunks, c = i - r * chunks;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < n_valid && c * 8 < dk) {
      const int tl = r / hb, hl = r - tl * hb;
      v = *reinterpret_cast<const uint4*>(q + (long long)(first + t0 + tl) * q_row_stride + (long long)(h0 + hl) * dk + c * 8);
    }
    *reinterpret_cast<uint4*>(q_s + r * ld + c * 8) = v;
  }
  if (dkp > dk)                             // the keys' channels past rank + rot, which no copy writes
    for (int i = tid; i < 2 * LM_KT; i += blockDim.x) *reinterpret_cast<uint4*>(k_s + i * ld + dk) = make_uint4(0u, 0u, 0u, 0u);
  // this lane's two rows of its row group
  const int g = lane >> 2, qd = lane & 3;
  int row_pos[2];
  bool row_ok[2];
  float m_run[2], l_run[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = rg * 16 + g + 8 * e;
    const int tl = r / hb, hl = r - tl * hb;
    row_ok[e] = r < n_valid;
    row_pos[e] = past + t0 + tl;
    const bool has_sink = row_ok[e] && sink != nullptr && split == 0;
    m_run[e] = has_sink ? sink[h0 + hl] * LOG2E : -INFINITY;
    l_run[e] = has_sink ? 1.f : 0.f;
  }
  float acc[2 * NP][4];
#pragma unroll
  for (int j = 0; j < 2 * NP; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
  const float scale_log2 = scale * LOG2E;
  const int last_pos = past + min(t0 + tq, n_new) - 1;
  const int n_tiles = last_pos / LM_KT + 1;
  // (`window` > 0: a row sees the last `window` positions up to its own; tiles before the first token's are skipped)
  const int tile_first = window > 0 ? max(0, past + t0 - window + 1) / LM_KT : 0;
  const int per = (n_tiles - tile_first + n_splits - 1) / n_splits;
  const int tile_lo = tile_first + split * per, tile_hi = min(n_tiles, tile_lo + per);
  const int row_chunks = dk / 8;
  auto load_tile = [&](int tile, int buf) {
    const int j0 = tile * LM_KT;
    __nv_bfloat16* dst = k_s + buf * LM_KT * ld;
    for (int i = tid; i < LM_KT * row_chunks; i += blockDim.x) {
      const int kk = i / row_chunks, c = i - kk * row_chunks;
      const int j = j0 + kk;
      const __nv_bfloat16* src = pool;
      int bytes = 0;
      if (j <= last_pos) {
        const int lp = j / page_size;
        const int page = table[(long long)seq * table_stride + (lp % table_len)];
        src = pool + ((long long)page * page_size + (j - lp * page_size)) * dk + c * 8;
        bytes = 16;
      }
      lm_cp_async16(ds_smem(dst + kk * ld + c * 8), src, bytes);
    }
    lm_cp_commit();
  };
  if (tile_lo < tile_hi) load_tile(tile_lo, 0);
  const unsigned q_addr = ds_smem(q_s + (rg * 16 + (lane & 15)) * ld + (lane >> 4) * 8);
  const unsigned p_addr = ds_smem(p_s + (rg * 16 + (lane & 15)) * LM_PLD + (lane >> 4) * 8);
  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int buf = (tile - tile_lo) & 1;
    lm_cp_wait_all();
    __syncthreads();          // the tile is there for everyone, and everyone is done with the other buffer
    if (tile + 1 < tile_hi) load_tile(tile + 1, buf ^ 1);
    const __nv_bfloat16* kt = k_s + buf * LM_KT * ld;
    const int j0 = tile * LM_KT;
    const int key_base = vw * (LM_KT / VW);
    float s[NT][4];
    if (active) {
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
      const unsigned k_addr = ds_smem(kt + (key_base + (lane & 7)) * ld + ((lane >> 3) & 1) * 8);
#pragma unroll 2
      for (int ks = 0; ks < dkp / 16; ++ks) {
        unsigned a[4];
        ds_ldmatrix_x4(a, q_addr + ks * 32);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          unsigned b[2];
          lm_ldmatrix_x2(b, k_addr + (unsigned)(n * 8 * ld * 2) + ks * 32);
          ds_mma(s[n], a[0], a[1], a[2], a[3], b[0], b[1]);
        }
      }
      // mask, scale; the warp's maximum per row
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + key_base + n * 8 + qd * 2 + (e & 1);
          const int rr = e >> 1;
          const float v = (row_ok[rr] && j <= row_pos[rr] && (window <= 0 || row_pos[rr] - j < window))
                              ? s[n][e] * scale_log2 : -INFINITY;
          s[n][e] = v;
          mx[rr] = fmaxf(mx[rr], v);
        }
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
        mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
        if (qd == 0) red_max[(rg * VW + vw) * 16 + g + 8 * rr] = mx[rr];
      }
    }
    __syncthreads();
    float corr[2] = {1.f, 1.f};
    if (active) {
      float ps[2] = {0.f, 0.f};
      float m_new[2];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        float m = m_run[rr];
#pragma unroll
        for (int v = 0; v < VW; ++v) m = fmaxf(m, red_max[(rg * VW + v) * 16 + g + 8 * rr]);
        m_new[rr] = m;
        corr[rr] = m == -INFINITY ? 1.f : ds_exp2(m_run[rr] - m);
        m_run[rr] = m;
      }
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p[e] = s[n][e] == -INFINITY ? 0.f : ds_exp2(s[n][e] - m_new[e >> 1]);
          ps[e >> 1] += p[e];
        }
        __nv_bfloat16* dst = p_s + (rg * 16 + g) * LM_PLD + key_base + n * 8 + qd * 2;
        *reinterpret_cast<unsigned*>(dst) = ds_pack(p[0], p[1]);
        *reinterpret_cast<unsigned*>(dst + 8 * LM_PLD) = ds_pack(p[2], p[3]);
      }
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        ps[rr] += __shfl_xor_sync(0xffffffffu, ps[rr], 1);
        ps[rr] += __shfl_xor_sync(0xffffffffu, ps[rr], 2);
        if (qd == 0) red_sum[(rg * VW + vw) * 16 + g + 8 * rr] = ps[rr];
      }
    }
    __syncthreads();
    if (active) {
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        float sum = 0.f;
#pragma unroll
        for (int v = 0; v < VW; ++v) sum += red_sum[(rg * VW + v) * 16 + g + 8 * rr];
        l_run[rr] = l_run[rr] * corr[rr] + sum;
      }
#pragma unroll
      for (int j = 0; j < 2 * NP; ++j) {
        acc[j][0] *= corr[0];
        acc[j][1] *= corr[0];
        acc[j][2] *= corr[1];
        acc[j][3] *= corr[1];
      }
      // value mix: the group's 16 x 32 weights times this warp's channels of the tile's rows
      const int ch_base = vw * vc;
      const int blk = lane >> 3;
      const unsigned v_addr = ds_smem(kt + ((blk & 1) * 8 + (lane & 7)) * ld + ch_base + (blk >> 1) * 8);
#pragma unroll
      for (int k2 = 0; k2 < LM_KT / 16; ++k2) {
        unsigned a[4];
        ds_ldmatrix_x4(a, p_addr + k2 * 32);
#pragma unroll
        for (int np = 0; np < NP; ++np) {
          if (np * 16 < vc) {
            unsigned b[4];
            ds_ldmatrix_x4_trans(b, v_addr + (unsigned)(k2 * 16 * ld * 2) + np * 32);
            ds_mma(acc[2 * np], a[0], a[1], a[2], a[3], b[0], b[1]);
            ds_mma(acc[2 * np + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
          }
        }
      }
    }
  }
  lm_cp_wait_all();
  if (!active) return;
  const int ch_base = vw * vc;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    if (!row_ok[rr]) continue;
    const int r = rg * 16 + g + 8 * rr;
    const int tl = r / hb, hl = r - tl * hb;
    const long long token = first + t0 + tl;
    const int head = h0 + hl;
    if (n_splits == 1) {
      const float inv = l_run[rr] > 0.f ? 1.f / l_run[rr] : 0.f;
      __nv_bfloat16* dst = out + token * out_row_stride + (long long)head * rank + ch_base;
#pragma unroll
      for (int j = 0; j < 2 * NP; ++j) {
        const int c = j * 8 + qd * 2;
        if (c < vc) *reinterpret_cast<unsigned*>(dst + c) = ds_pack(acc[j][2 * rr] * inv, acc[j][2 * rr + 1] * inv);
      }
    } else {
      float* dst = part + ((token * n_heads + head) * n_splits + split) * (rank + 2);
#pragma unroll
      for (int j = 0; j < 2 * NP; ++j) {
        const int c = j * 8 + qd * 2;
        if (c < vc) {
          dst[ch_base + c] = acc[j][2 * rr];
          dst[ch_base + c + 1] = acc[j][2 * rr + 1];
        }
      }
      if (vw == 0 && qd == 0) {
        dst[rank] = m_run[rr] == -INFINITY ? -INFINITY : m_run[rr] * 0.6931471805599453f;   // back to natural logarithms
        dst[rank + 1] = l_run[rr];
      }
    }
  }
}

// 0: the shape is not taken (the 32-bit kernel runs it); else the warps per row group.
static int lm_value_warps(int rank, int rot) {
  if ((rank + rot) % 8 != 0 || rank > 512) return 0;
  const int vw = rank <= 128 ? 1 : rank <= 256 ? 2 : 4;
  if (rank % (8 * vw) != 0) return 0;
  return vw;
}

int latent_attention_mma_rows() { return LM_BM; }
bool latent_attention_mma_supports(int rank, int rot) { return lm_value_warps(rank, rot) != 0; }

int launch_latent_attention_mma(const __nv_bfloat16* q, long long q_row_stride, const __nv_bfloat16* pool, const int* table,
                                int table_stride, int table_len, int page_size, const int* seq_start, const int* past_len,
                                const float* sink, __nv_bfloat16* out, long long out_row_stride, float* part, int n_seqs,
                                int max_new, int n_heads, int rank, int rot, float scale, int n_splits, int window,
                                cudaStream_t stream) {
  const int vw = lm_value_warps(rank, rot);
  BT_CHECK(vw != 0, "latent_attention: rank %d, rot %d is no shape of the tensor-core kernel", rank, rot);
  BT_CHECK(((unsigned long long)q % 16) == 0 && ((unsigned long long)pool % 16) == 0 && (q_row_stride % 8) == 0 &&
           ((unsigned long long)out % 4) == 0, "latent_attention: queries and cache rows must lie on 16-byte boundaries");
  const int dk = rank + rot, dkp = (dk + 15) & ~15, ld = dkp + LM_PAD;
  const int vc = rank / vw;
  const int hb = n_heads < LM_BM ? n_heads : LM_BM;
  const int tq = LM_BM / hb;
  const int head_tiles = (n_heads + hb - 1) / hb;
  const int token_tiles = (max_new + tq - 1) / tq;
  const size_t smem = (size_t)(LM_BM + 2 * LM_KT) * ld * 2 + 4 * 16 * LM_PLD * 2 + 2 * 4 * vw * 16 * sizeof(float);
  BT_CHECK(smem <= 227 * 1024, "latent_attention: rank + rot = %d needs %zu bytes of shared memory", dk, smem);
  const dim3 grid(token_tiles * head_tiles, n_splits, n_seqs), block(128 * vw);
#define BT_LM(VW, VCT)                                                                                               \
  do {                                                                                                               \
    auto kernel = latent_attention_mma_kernel<VW, VCT>;                                                              \
    static size_t reserved = 0;   /* (the attribute is set again only when a call needs more than any before) */     \
    if (smem > 48 * 1024 && smem > reserved) {                                                                       \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
      BT_CHECK(e == cudaSuccess, "latent_attention: cannot reserve %zu bytes of shared memory", smem);               \
      reserved = smem;                                                                                               \
    }                                                                                                                \
    BT_PDL_OK("latent_attention_mma",                                                                                \
              launch_pdl(kernel, grid, block, smem, stream, 1, q, q_row_stride, pool, table, table_stride, table_len, \
                         page_size, seq_start, past_len, sink, out, out_row_stride, part, n_heads, hb, tq, head_tiles, \
                         rank, rot, scale, n_splits, window));                                                       \
  } while (0)
  if (vw == 1 && vc <= 32) BT_LM(1, 32);
  else if (vw == 1 && vc <= 64) BT_LM(1, 64);
  else if (vw == 1) BT_LM(1, 128);
  else if (vw == 2) BT_LM(2, 128);
  else BT_LM(4, 128);
#undef BT_LM
  return 0;
}

}  // namespace bt
