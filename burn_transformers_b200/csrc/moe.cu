// Routed experts: the router with its choice of experts, the sorting of (token, choice) pairs by expert, the experts'
// two products over the sorted rows, and the weighted sum back into the stream.
//
//   moe_route    per token: z = W_r x in 32-bit, s = sigmoid(z); experts lie in `n_groups` equal groups of neighbours, a
//                group's score is the sum of its two largest s, only the `keep` best groups may give experts; the `top`
//                largest s among those are chosen (equal scores: the lower index); weights s / (sum of the chosen + 1e-20)
//                * scale.  With `softmax` the scores are softmax(z) over all experts instead; `choice_bias` [E] is added
//                to the scores for the choice only; without `normalise` the weights are the chosen scores as they are.
//   moe_sort     counts the pairs per expert, gives each pair a row in expert order, and numbers the row tiles
//                (tiles never straddle two experts).
//   moe_expert_in   hidden[r] = pair rule(gate_e x, up_e x) for the rows of expert e (x gathered by the pair's token), or,
//                   for experts without a gate, act(up_e x)
//   moe_expert_out  part[r] = weight(r) * down_e hidden[r]   (32-bit)
//   moe_combine  stream[t] += sum over the token's pairs, in the order of its choices: no atomics, a fixed order.  A pair
//                whose expert's number is `n_stored` or more names an expert without tensors that hands its input on: the
//                pair adds weight * input[t].
//
// The products exist as 32-bit multiply-adds (float32, and every shape), on tensor cores (bfloat16, mma.sync m16n8k16
// with 32-bit accumulators, K a multiple of 8) and, for steps with few rows an expert, as a kernel that streams every
// expert's weights once (bfloat16).  A row's result never depends on its neighbours in the tile.
#include "common.cuh"

namespace bt {

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

constexpr int ROUTE_WARPS = 4;

// A 16-byte piece of a row as 32-bit numbers.
__device__ __forceinline__ void load_piece(const float* p, float (&o)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
__device__ __forceinline__ void load_piece(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ void unpack_piece(const uint4& v, float (&o)[4]) {
  o[0] = __uint_as_float(v.x); o[1] = __uint_as_float(v.y); o[2] = __uint_as_float(v.z); o[3] = __uint_as_float(v.w);
}
__device__ __forceinline__ void unpack_piece(const uint4& v, float (&o)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}

// NP > 0: the token's row is whole 16-byte pieces, at most NP a lane; the lane keeps them in registers and asks for the
// pieces of four experts' rows at once, so that a token costs a few trips to memory, not one per expert and piece.
template <typename T, int NP>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const T* __restrict__ x, long long x_row_stride, const T* __restrict__ router, int n_tokens, int K, int E,
                 int top, int n_groups, int keep, float scale, int softmax, const float* __restrict__ choice_bias,
                 int normalise, int* __restrict__ ids, float* __restrict__ weights) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* score = sm + (size_t)warp * 3 * E;   // [E] sigmoid scores
  float* cand = score + E;                    // [E] scores still to choose from (-inf: not allowed, or taken)
  float* group = cand + E;                    // [n_groups] group scores
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= n_tokens) return;
  const T* row = x + (long long)t * x_row_stride;
  constexpr int V = 16 / (int)sizeof(T), EB = 4;
  if (NP > 0) {
    float xv[NP > 0 ? NP : 1][V];
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      const int k = (lane + 32 * i) * V;
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (k < K) raw = *reinterpret_cast<const uint4*>(row + k);
      unpack_piece(raw, xv[i]);
    }
    for (int e0 = 0; e0 < E; e0 += EB) {
      uint4 raw[EB][NP > 0 ? NP : 1];
#pragma unroll
      for (int j = 0; j < EB; ++j)
#pragma unroll
        for (int i = 0; i < NP; ++i) {
          const int k = (lane + 32 * i) * V;
          raw[j][i] = (e0 + j < E && k < K) ? *reinterpret_cast<const uint4*>(router + (long long)(e0 + j) * K + k)
                                            : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
      for (int j = 0; j < EB; ++j) {
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < NP; ++i) {
          float wv[V];
          unpack_piece(raw[j][i], wv);
#pragma unroll
          for (int u = 0; u < V; ++u) acc = fmaf(xv[i][u], wv[u], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0 && e0 + j < E) score[e0 + j] = softmax ? acc : 1.f / (1.f + expf(-acc));
      }
    }
  } else {
    for (int e0 = 0; e0 < E; e0 += EB) {
      float acc[EB] = {0.f, 0.f, 0.f, 0.f};
      for (int k = lane; k < K; k += 32) {
        const float xs = to_float(row[k]);
#pragma unroll
        for (int j = 0; j < EB; ++j)
          if (e0 + j < E) acc[j] = fmaf(xs, to_float(router[(long long)(e0 + j) * K + k]), acc[j]);
      }
#pragma unroll
      for (int j = 0; j < EB; ++j) {
        const float z = warp_sum(acc[j]);
        if (lane == 0 && e0 + j < E) score[e0 + j] = softmax ? z : 1.f / (1.f + expf(-z));
      }
    }
  }
  __syncwarp();
  if (softmax) {
    float top_z = -INFINITY;
    for (int e = lane; e < E; e += 32) top_z = fmaxf(top_z, score[e]);
    top_z = warp_max(top_z);
    float denom = 0.f;
    for (int e = lane; e < E; e += 32) denom += expf(score[e] - top_z);
    denom = warp_sum(denom);
    for (int e = lane; e < E; e += 32) score[e] = expf(score[e] - top_z) / denom;
    __syncwarp();
  }
  for (int e = lane; e < E; e += 32) cand[e] = score[e] + (choice_bias != nullptr ? choice_bias[e] : 0.f);
  if (keep < n_groups) {
    const int size = E / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float a = -1.f, b = -1.f;               // the two largest of the group
      for (int e = g * size; e < (g + 1) * size; ++e) {
        const float s = score[e];
        if (s > a) { b = a; a = s; } else if (s > b) { b = s; }
      }
      group[g] = a + (b >= 0.f ? b : 0.f);
    }
    __syncwarp();
    // take `keep` groups out (marking them), then close the experts of the groups that stayed
    for (int r = 0; r < keep; ++r) {
      float v = -INFINITY;
      int i = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32)
        if (group[g] > v) { v = group[g]; i = g; }
      warp_argmax(v, i);
      __syncwarp();
      if (lane == 0) group[i] = -INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (group[e / size] != -INFINITY) cand[e] = -INFINITY;
  }
  __syncwarp();
  float sum = 0.f;
  for (int r = 0; r < top; ++r) {
    float v = -INFINITY;
    int i = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (cand[e] > v) { v = cand[e]; i = e; }
    warp_argmax(v, i);
    __syncwarp();
    v = score[i];       // (the weight is the score itself, whatever was added for the choice)
    if (lane == 0) {
      cand[i] = -INFINITY;
      ids[(long long)t * top + r] = i;
      weights[(long long)t * top + r] = v;
    }
    sum += v;
    __syncwarp();
  }
  if (normalise && lane < top) {
    const long long at = (long long)t * top + lane;
    weights[at] = weights[at] / (sum + 1e-20f) * scale;
  }
}

// One block.  offsets[e]: first sorted row of expert e (offsets[E] = all rows); tile_first[e]: first row tile of expert e
// (tile_first[E] = all tiles); order[r]: the pair (token * top + choice) that lies in sorted row r; place[pair]: its row.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int total, int E, int tile_rows, int* __restrict__ offsets,
                int* __restrict__ tile_first, int* __restrict__ order, int* __restrict__ place) {
  extern __shared__ int ism[];
  int* count = ism;         // [E]
  int* cursor = ism + E;    // [E]
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < total; i += blockDim.x) atomicAdd(&count[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int rows = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = rows;
      tile_first[e] = tiles;
      cursor[e] = rows;
      rows += count[e];
      tiles += (count[e] + tile_rows - 1) / tile_rows;
    }
    offsets[E] = rows;
    tile_first[E] = tiles;
  }
  __syncthreads();
  // lanes of a warp that hold the same expert take consecutive rows from one atomic; which pair gets which of an
  // expert's rows does not matter: a row's result does not depend on its place
  for (int base = 0; base < total; base += blockDim.x) {
    const int i = base + threadIdx.x;
    if (i < total) {
      const int e = ids[i];
      const unsigned same = __match_any_sync(__activemask(), e);
      const int rank = __popc(same & ((1u << (threadIdx.x & 31)) - 1));
      int first = 0;
      if (rank == 0) first = atomicAdd(&cursor[e], __popc(same));
      first = __shfl_sync(same, first, __ffs(same) - 1);
      order[first + rank] = i;
      place[i] = first + rank;
    }
  }
}

// Which expert and which of its rows a row tile holds: the last e with tile_first[e] <= tile.
__device__ __forceinline__ bool moe_tile(const int* __restrict__ offsets, const int* __restrict__ tile_first, int E,
                                         int tile, int tile_rows, int& expert, int& row0, int& rows) {
  if (tile >= tile_first[E]) return false;
  int lo = 0, hi = E - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tile_first[mid] <= tile) lo = mid; else hi = mid - 1;
  }
  expert = lo;
  row0 = offsets[lo] + (tile - tile_first[lo]) * tile_rows;
  rows = min(tile_rows, offsets[lo + 1] - row0);
  return true;
}

// ---- the products as 32-bit multiply-adds ---------------------------------------------------------------------------
constexpr int MS_BM = 32, MS_BN = 64, MS_BK = 32;

struct MoeArgs {
  const int* offsets;
  const int* tile_first;
  const int* order;
  const float* pair_weight;   // [pairs] (second product)
  int E, top, K, N, act;
  float limit;
  long long a_row_stride;
};

// MODE 1: hidden[r, j] = pair(gate_e[j] . x, up_e[j] . x), w: [E][2N][K];  MODE 2 (experts without a gate): hidden[r, j] =
// act(up_e[j] . x), w: [E][N][K];  MODE 0: part[r, c] = weight * (down_e[c] . hidden[r]), w: [E][N][K].
constexpr int kMoeOut = 0, kMoeInPair = 1, kMoeInPlain = 2;

template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_expert_simt_kernel(const T* __restrict__ a, const T* __restrict__ w, void* __restrict__ out, MoeArgs p) {
  constexpr bool IN = MODE != kMoeOut, PAIR = MODE == kMoeInPair;
  __shared__ float a_s[MS_BK][MS_BM + 1];
  __shared__ float w_s[PAIR ? 2 : 1][MS_BK][MS_BN + 1];
  __shared__ int src_row[MS_BM];
  pdl_trigger();
  pdl_wait();
  int expert, row0, rows;
  if (!moe_tile(p.offsets, p.tile_first, p.E, blockIdx.y, MS_BM, expert, row0, rows)) return;
  const int n0 = blockIdx.x * MS_BN;
  if (threadIdx.x < MS_BM) {
    const int r = row0 + threadIdx.x;
    src_row[threadIdx.x] = threadIdx.x < rows ? (IN ? p.order[r] / p.top : r) : -1;
  }
  __syncthreads();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 4 columns, 2 rows a thread
  float acc[PAIR ? 2 : 1][2][4] = {};
  const T* w_e = w + (long long)expert * (PAIR ? 2 : 1) * p.N * p.K;
  for (int k0 = 0; k0 < p.K; k0 += MS_BK) {
    for (int i = threadIdx.x; i < MS_BM * MS_BK; i += 256) {
      const int r = i / MS_BK, k = i - r * MS_BK;
      const int src = src_row[r];
      a_s[k][r] = src >= 0 && k0 + k < p.K ? to_float(a[(long long)src * p.a_row_stride + k0 + k]) : 0.f;
    }
    for (int i = threadIdx.x; i < MS_BN * MS_BK; i += 256) {
      const int n = i / MS_BK, k = i - n * MS_BK;
      const bool in = n0 + n < p.N && k0 + k < p.K;
      w_s[0][k][n] = in ? to_float(w_e[(long long)(n0 + n) * p.K + k0 + k]) : 0.f;
      if (PAIR) w_s[PAIR ? 1 : 0][k][n] = in ? to_float(w_e[(long long)(p.N + n0 + n) * p.K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < MS_BK; ++k) {
      const float a0 = a_s[k][ty * 2], a1 = a_s[k][ty * 2 + 1];
#pragma unroll
      for (int h = 0; h < (PAIR ? 2 : 1); ++h)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float b = w_s[h][k][tx * 4 + c];
          acc[h][0][c] = fmaf(a0, b, acc[h][0][c]);
          acc[h][1][c] = fmaf(a1, b, acc[h][1][c]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int rl = ty * 2 + i;
    if (rl >= rows) continue;
    const long long r = row0 + rl;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int n = n0 + tx * 4 + c;
      if (n >= p.N) continue;
      if (IN)
        reinterpret_cast<T*>(out)[r * p.N + n] = from_float<T>(
            PAIR ? gated_pair(acc[0][i][c], acc[PAIR ? 1 : 0][i][c], p.act, p.limit) : apply_activation(acc[0][i][c], p.act));
      else
        reinterpret_cast<float*>(out)[r * p.N + n] = acc[0][i][c] * p.pair_weight[p.order[r]];
    }
  }
}

// ---- the products on tensor cores (bfloat16) -----------------------------------------------------------------------
// A block: 32 rows x 64 columns (both halves of the pair for the first product), 4 warps, each 32 rows x 16 columns; K in
// pieces of 32 through a ring of three shared-memory stages filled by cp.async (rows padded to 40 elements: fragment
// loads fall into different banks).
constexpr int MM_BM = 32, MM_BN = 64, MM_BK = 32, MM_LD = MM_BK + 8, MM_STAGES = 3;

// 16 bytes from global to shared memory without passing registers; `real` false copies no source bytes and fills zeros.
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool real) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = real ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int MODE>
__global__ void __launch_bounds__(128)
moe_expert_mma_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w, void* __restrict__ out,
                      MoeArgs p) {
  constexpr bool IN = MODE != kMoeOut, PAIR = MODE == kMoeInPair;
  constexpr int HALVES = PAIR ? 2 : 1;
  __shared__ __align__(16) __nv_bfloat16 a_s[MM_STAGES][MM_BM][MM_LD];
  __shared__ __align__(16) __nv_bfloat16 w_s[MM_STAGES][HALVES][MM_BN][MM_LD];
  __shared__ int src_row[MM_BM];
  pdl_trigger();
  pdl_wait();
  int expert, row0, rows;
  if (!moe_tile(p.offsets, p.tile_first, p.E, blockIdx.y, MM_BM, expert, row0, rows)) return;
  const int n0 = blockIdx.x * MM_BN;
  if (threadIdx.x < MM_BM) {
    const int r = row0 + threadIdx.x;
    src_row[threadIdx.x] = threadIdx.x < rows ? (IN ? p.order[r] / p.top : r) : -1;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  float acc[HALVES][2][2][4] = {};      // [half][m tile][n tile][fragment]
  const __nv_bfloat16* w_e = w + (long long)expert * HALVES * p.N * p.K;
  // 16-byte pieces, 4 a row: a thread moves one piece of the rows and two (four, with both halves) of the weights per
  // K piece, by cp.async into a ring of MM_STAGES K pieces: while one piece is multiplied, the next two are in flight
  // (a piece outside the rows, the columns or K is filled with zeros: a copy of no source bytes)
  const int pr = threadIdx.x >> 2, pc = (threadIdx.x & 3) * 8;
  const int a_src = src_row[pr];
  auto issue = [&](int stage, int k0) {
    if (k0 < p.K) {
      const bool in_k = k0 + pc < p.K;
      const bool ok = a_src >= 0 && in_k;
      cp_async_16(&a_s[stage][pr][pc], ok ? a + (long long)a_src * p.a_row_stride + k0 + pc : a, ok);
#pragma unroll
      for (int h = 0; h < HALVES; ++h)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int n = n0 + pr + 32 * j;
          const bool okw = n < p.N && in_k;
          cp_async_16(&w_s[stage][h][pr + 32 * j][pc], okw ? w_e + (long long)(h * p.N + n) * p.K + k0 + pc : w_e, okw);
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");      // (an empty group keeps the count of groups in step)
  };
#pragma unroll
  for (int st = 0; st < MM_STAGES - 1; ++st) issue(st, st * MM_BK);
  int stage = 0;
  for (int k0 = 0; k0 < p.K; k0 += MM_BK) {
    asm volatile("cp.async.wait_group %0;" ::"n"(MM_STAGES - 2) : "memory");
    __syncthreads();      // this piece has landed for every thread, and the piece multiplied last is free again
    issue((stage + MM_STAGES - 1) % MM_STAGES, k0 + (MM_STAGES - 1) * MM_BK);
#pragma unroll
    for (int kk = 0; kk < MM_BK; kk += 16) {
      uint32_t af[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const __nv_bfloat16* base = &a_s[stage][mt * 16 + gid][kk + tig * 2];
        af[mt][0] = *reinterpret_cast<const uint32_t*>(base);
        af[mt][1] = *reinterpret_cast<const uint32_t*>(base + 8 * MM_LD);
        af[mt][2] = *reinterpret_cast<const uint32_t*>(base + 8);
        af[mt][3] = *reinterpret_cast<const uint32_t*>(base + 8 * MM_LD + 8);
      }
#pragma unroll
      for (int h = 0; h < HALVES; ++h)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const __nv_bfloat16* base = &w_s[stage][h][warp * 16 + nt * 8 + gid][kk + tig * 2];
          uint32_t bf[2];
          bf[0] = *reinterpret_cast<const uint32_t*>(base);
          bf[1] = *reinterpret_cast<const uint32_t*>(base + 8);
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) mma_bf16_16816(acc[h][mt][nt], af[mt], bf);
        }
    }
    stage = (stage + 1) % MM_STAGES;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int rl = mt * 16 + gid + half * 8;
      if (rl >= rows) continue;
      const long long r = row0 + rl;
      const float scale = IN ? 1.f : p.pair_weight[p.order[r]];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + warp * 16 + nt * 8 + tig * 2 + c;
          if (n >= p.N) continue;
          const float v = acc[0][mt][nt][half * 2 + c];
          if (IN)
            reinterpret_cast<__nv_bfloat16*>(out)[r * p.N + n] =
                __float2bfloat16_rn(PAIR ? gated_pair(v, acc[PAIR ? 1 : 0][mt][nt][half * 2 + c], p.act, p.limit)
                                         : apply_activation(v, p.act));
          else
            reinterpret_cast<float*>(out)[r * p.N + n] = v * scale;
        }
    }
}

// ---- the products for few rows an expert (decode steps, bfloat16) ---------------------------------------------------
// A block: one expert and 8 output columns (each of 4 warps two columns; for the first product the gate's and up's rows
// of a column together).  The expert's rows, 8 at a time, lie in shared memory; a warp streams its columns' weight
// rows once per 8 rows, a lane 16-byte pieces of K, sums in 32-bit, and the lanes' sums meet by shuffles.  Every weight
// byte is read by one warp; a block whose expert got no row ends at once.
constexpr int MF_ROWS = 8, MF_COLS = 8, MF_KC = 2048;

template <int MODE>
__global__ void __launch_bounds__(128)
moe_expert_few_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w, void* __restrict__ out,
                      MoeArgs p) {
  constexpr bool IN = MODE != kMoeOut, PAIR = MODE == kMoeInPair;
  __shared__ __align__(16) __nv_bfloat16 x_s[MF_ROWS][MF_KC];
  pdl_trigger();
  pdl_wait();
  const int expert = blockIdx.y;
  const int first = p.offsets[expert], count = p.offsets[expert + 1] - first;
  if (count == 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * MF_COLS + warp * 2;
  const __nv_bfloat16* w_e = w + (long long)expert * (PAIR ? 2 : 1) * p.N * p.K;
  for (int r0 = 0; r0 < count; r0 += MF_ROWS) {
    const int rows = min(MF_ROWS, count - r0);
    float acc[PAIR ? 2 : 1][2][MF_ROWS] = {};
    for (int k0 = 0; k0 < p.K; k0 += MF_KC) {
      const int kc = min(MF_KC, p.K - k0);
      __syncthreads();
      for (int i = threadIdx.x; i < MF_ROWS * (kc / 8); i += 128) {
        const int r = i / (kc / 8), c = (i - r * (kc / 8)) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) {
          const long long src = IN ? p.order[first + r0 + r] / p.top : first + r0 + r;
          v = *reinterpret_cast<const uint4*>(a + src * p.a_row_stride + k0 + c);
        }
        *reinterpret_cast<uint4*>(&x_s[r][c]) = v;
      }
      __syncthreads();
#pragma unroll
      for (int col = 0; col < 2; ++col) {
        const int n = n0 + col;
        if (n >= p.N) continue;
        for (int k = lane * 8; k < kc; k += 256) {
          float wv[PAIR ? 2 : 1][8];
          load_piece(w_e + (long long)n * p.K + k0 + k, wv[0]);
          if (PAIR) load_piece(w_e + (long long)(p.N + n) * p.K + k0 + k, wv[PAIR ? 1 : 0]);
#pragma unroll
          for (int r = 0; r < MF_ROWS; ++r) {
            float xv[8];
            load_piece(&x_s[r][k], xv);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              acc[0][col][r] = fmaf(xv[u], wv[0][u], acc[0][col][r]);
              if (PAIR) acc[PAIR ? 1 : 0][col][r] = fmaf(xv[u], wv[PAIR ? 1 : 0][u], acc[PAIR ? 1 : 0][col][r]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int col = 0; col < 2; ++col)
#pragma unroll
      for (int r = 0; r < MF_ROWS; ++r) {
        const float g = warp_sum(acc[0][col][r]);
        const float u = PAIR ? warp_sum(acc[PAIR ? 1 : 0][col][r]) : 0.f;
        const int n = n0 + col;
        if (lane == 0 && r < rows && n < p.N) {
          const long long row = first + r0 + r;
          if (IN)
            reinterpret_cast<__nv_bfloat16*>(out)[row * p.N + n] =
                __float2bfloat16_rn(PAIR ? gated_pair(g, u, p.act, p.limit) : apply_activation(g, p.act));
          else
            reinterpret_cast<float*>(out)[row * p.N + n] = g * p.pair_weight[p.order[row]];
        }
      }
  }
}

// stream[t, c] += sum_j part[place[t * top + j], c] (`store`: =, the rows are written, not added to); a pair whose expert
// is `n_stored` or more adds weight * input[t, c] instead (`ids` null: every pair has a row in `part`)
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ part, const int* __restrict__ place, float* __restrict__ stream,
                   long long n_tokens, int top, int width, const int* __restrict__ ids, const float* __restrict__ weights,
                   const float* __restrict__ input, int n_stored, int store) {
  pdl_trigger();
  pdl_wait();
  const long long total = n_tokens * width;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / width;
    const int c = (int)(i - t * width);
    float sum = 0.f;
    for (int j = 0; j < top; ++j) {
      if (ids != nullptr && ids[t * top + j] >= n_stored) sum = fmaf(weights[t * top + j], input[i], sum);
      else sum += part[(long long)place[t * top + j] * width + c];
    }
    stream[i] = store ? sum : stream[i] + sum;      // (`store`: the rows hold nothing yet)
  }
}

}  // namespace bt

extern "C" int bt_moe_route(const void* x, long long x_row_stride, const void* router, int n_tokens, int K, int E, int top,
                            int n_groups, int keep, float scale, int softmax, const float* choice_bias, int normalise,
                            int* ids, float* weights, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_tokens >= 0 && K > 0 && E > 0 && E <= 1024 && top > 0 && top <= 32 && n_groups > 0 && E % n_groups == 0 &&
               keep > 0 && keep <= n_groups && top <= keep * (E / n_groups),
           "moe_route: bad sizes experts=%d (up to 1024) top=%d (up to 32) groups=%d keep=%d", E, top, n_groups, keep);
  if (n_tokens == 0) return 0;
  const dim3 grid((n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), block(ROUTE_WARPS * 32);
  const size_t smem = (size_t)ROUTE_WARPS * 3 * E * sizeof(float);
  // pieces of 16 bytes a lane holds of a token's row: 1, 2 or 4 (rows of up to 128 pieces); 0: element by element
  auto pieces_of = [&](int elem) {
    const int v = 16 / elem;
    if (K % v || x_row_stride % v || (unsigned long long)x % 16 || (unsigned long long)router % 16) return 0;
    const int per_lane = (K / v + 31) / 32;
    return per_lane <= 1 ? 1 : per_lane <= 2 ? 2 : per_lane <= 4 ? 4 : 0;
  };
#define BT_ROUTE(T, NP)                                                                                              \
  BT_PDL_OK("moe_route", launch_pdl(moe_route_kernel<T, NP>, grid, block, smem, stream, 1, (const T*)x, x_row_stride, \
                                    (const T*)router, n_tokens, K, E, top, n_groups, keep, scale, softmax, choice_bias, \
                                    normalise, ids, weights))
  if (dtype == kF32) {
    const int np = pieces_of(4);
    if (np == 1) BT_ROUTE(float, 1); else if (np == 2) BT_ROUTE(float, 2); else if (np == 4) BT_ROUTE(float, 4);
    else BT_ROUTE(float, 0);
  } else if (dtype == kBF16) {
    const int np = pieces_of(2);
    if (np == 1) BT_ROUTE(__nv_bfloat16, 1); else if (np == 2) BT_ROUTE(__nv_bfloat16, 2);
    else if (np == 4) BT_ROUTE(__nv_bfloat16, 4); else BT_ROUTE(__nv_bfloat16, 0);
  } else {
    return fail("moe_route: unknown dtype %d", dtype);
  }
#undef BT_ROUTE
  return 0;
}

extern "C" int bt_moe_tile_rows() { return bt::MS_BM; }

extern "C" int bt_moe_sort(const int* ids, int total, int E, int* offsets, int* tile_first, int* order, int* place,
                           cudaStream_t stream) {
  using namespace bt;
  static_assert(MS_BM == MM_BM, "both product kernels read the same row tiles");
  BT_CHECK(total >= 0 && E > 0 && E <= 4096, "moe_sort: bad sizes pairs=%d experts=%d", total, E);
  BT_PDL_OK("moe_sort", launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, 1, ids,
                                   total, E, MS_BM, offsets, tile_first, order, place));
  return 0;
}

// first: 1 = the experts' first product (a: the tokens' rows [tokens, K]; w: [E][2N][K]; out: [pairs, N] of the
// compute type), 2 = the first product of experts without a gate (w: [E][N][K]; out = act(product)), 0 = the second (a:
// [pairs, K]; w: [E][N][K]; out: [pairs, N] 32-bit, times the pair's weight).  E counts the experts with tensors; the
// sorted rows of pairs with a higher number lie behind theirs and are left alone.
extern "C" int bt_moe_expert(int first, const void* a, long long a_row_stride, const void* w, void* out,
                             const int* offsets, const int* tile_first, const int* order, const float* pair_weight,
                             int pairs, int E, int top, int K, int N, int act, float limit, int tensor_cores, int dtype,
                             cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(pairs >= 0 && E > 0 && top > 0 && K > 0 && N > 0 && first >= 0 && first <= 2,
           "moe_expert: bad sizes pairs=%d experts=%d K=%d N=%d", pairs, E, K, N);
  if (pairs == 0) return 0;
  MoeArgs p;
  p.offsets = offsets; p.tile_first = tile_first; p.order = order; p.pair_weight = pair_weight;
  p.E = E; p.top = top; p.K = K; p.N = N; p.act = act; p.limit = limit; p.a_row_stride = a_row_stride;
  const int tiles = (pairs + MS_BM - 1) / MS_BM + E;      // no more row tiles than this, however the pairs fall
  BT_CHECK(tiles <= 65535, "moe_expert: %d pairs are more row tiles than a launch takes", pairs);
  const dim3 grid((N + MS_BN - 1) / MS_BN, tiles);
  const bool pieces = dtype == kBF16 && K % 8 == 0 && a_row_stride % 8 == 0 && (unsigned long long)a % 16 == 0 &&
                      (unsigned long long)w % 16 == 0;
  if (pieces && tensor_cores && pairs <= 16 * E && E <= 65535) {
    // few rows an expert (a decode step): every expert's weights streamed once per 8 of its rows
    const dim3 few((N + MF_COLS - 1) / MF_COLS, E);
    if (first == kMoeInPair)
      BT_PDL_OK("moe_expert", launch_pdl(moe_expert_few_kernel<kMoeInPair>, few, dim3(128), 0, stream, 1,
                                         (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, out, p));
    else if (first == kMoeInPlain)
      BT_PDL_OK("moe_expert", launch_pdl(moe_expert_few_kernel<kMoeInPlain>, few, dim3(128), 0, stream, 1,
                                         (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, out, p));
    else
      BT_PDL_OK("moe_expert", launch_pdl(moe_expert_few_kernel<kMoeOut>, few, dim3(128), 0, stream, 1,
                                         (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, out, p));
    return 0;
  }
  if (dtype == kBF16 && tensor_cores && K % 8 == 0 && a_row_stride % 8 == 0 && (unsigned long long)a % 16 == 0 &&
      (unsigned long long)w % 16 == 0) {
    if (first == kMoeInPair)
      BT_PDL_OK("moe_expert", launch_pdl(moe_expert_mma_kernel<kMoeInPair>, grid, dim3(128), 0, stream, 1,
                                         (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, out, p));
    else if (first == kMoeInPlain)
      BT_PDL_OK("moe_expert", launch_pdl(moe_expert_mma_kernel<kMoeInPlain>, grid, dim3(128), 0, stream, 1,
                                         (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, out, p));
    else
      BT_PDL_OK("moe_expert", launch_pdl(moe_expert_mma_kernel<kMoeOut>, grid, dim3(128), 0, stream, 1,
                                         (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, out, p));
    return 0;
  }
#define BT_MOE(T, FIRST) \
  BT_PDL_OK("moe_expert", launch_pdl(moe_expert_simt_kernel<T, FIRST>, grid, dim3(256), 0, stream, 1, (const T*)a, (const T*)w, out, p))
#define BT_MOE_MODES(T)                                                                          \
  do {                                                                                           \
    if (first == kMoeInPair) BT_MOE(T, kMoeInPair); else if (first == kMoeInPlain) BT_MOE(T, kMoeInPlain); \
    else BT_MOE(T, kMoeOut);                                                                     \
  } while (0)
  if (dtype == kF32) BT_MOE_MODES(float);
  else if (dtype == kBF16) BT_MOE_MODES(__nv_bfloat16);
  else return fail("moe_expert: unknown dtype %d", dtype);
#undef BT_MOE_MODES
#undef BT_MOE
  return 0;
}

extern "C" int bt_moe_combine(const float* part, const int* place, float* stream_rows, long long n_tokens, int top,
                              int width, const int* ids, const float* weights, const float* input, int n_stored,
                              int store, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_tokens >= 0 && top > 0 && width > 0, "moe_combine: bad sizes");
  BT_CHECK(ids == nullptr || (weights != nullptr && input != nullptr), "moe_combine: pairs that hand the input on need weights and the input");
  if (n_tokens == 0) return 0;
  const long long total = n_tokens * width;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  BT_PDL_OK("moe_combine", launch_pdl(moe_combine_kernel, dim3(blocks), dim3(256), 0, stream, 1, part, place, stream_rows,
                                      n_tokens, top, width, ids, weights, input, n_stored, store));
  return 0;
}
