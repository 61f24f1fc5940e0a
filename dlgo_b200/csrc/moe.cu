// Routed experts (mixture of experts): router, plan, grouped contractions, combine.
//
// 1. moe_router:   z = Wr h in fp32 (Wr is kept in fp32), scores s = softmax(z) (or sigmoid(z)) over all
//                  router outputs, choice scores c = s + correction, group-limited choice of `top` outputs
//                  (outputs form `groups` equal groups of neighbours; a group's score is its largest choice
//                  score; only outputs of the `keep` best groups can be chosen, the others count as minus
//                  infinity), weights = the chosen outputs' s (optionally renormalised).  A bias on the logits
//                  (`zbias`, one number per output) is part of z: it moves scores and weights alike.  A further row of Wr
//                  (`has_gate`) gives a per-token gate sigmoid(w_g . h) for a shared expert.
// 2. moe_plan:     (token, choice) pairs sorted by expert: offsets per expert, the sorted pair list, and a list
//                  of row tiles (expert, first row), all on the device: nothing returns to the host, so the
//                  step can be captured in a CUDA graph.  Outputs at or beyond `n_experts` (identity experts)
//                  hold no tensors and enter no list.
// 3. moe_gemm:     out[row] = act(A[row] . W[expert]^T) tile by tile, rows gathered / scattered through the
//                  pair list.  Few rows per expert (decode): tiles of 8 rows, a warp per output, the expert's
//                  weight streamed once with 16-byte loads.  Many rows (prompts): 64 x 64 tiles on the fp32
//                  pipes, one running sum per output in k order.
// 4. moe_combine:  y[t] += sum_k weight[t][k] * (expert output of pair (t, k), or h[t] for an identity expert)
//                  + gate[t] * shared[t], pairs in the order they were chosen.
//
// A row's result never depends on which other rows are in its tile or launch.
#include "common.cuh"

#include <math_constants.h>

namespace dlgo {

enum { ACT_NONE = 0, ACT_RELU2 = 1, ACT_SILU = 2, ACT_GELU_TANH = 3 };

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case ACT_RELU2: { const float r = fmaxf(v, 0.f); return r * r; }
    case ACT_SILU: return v / (1.f + expf(-v));
    case ACT_GELU_TANH: return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    default: return v;
  }
}

// ------------------------------------------------------------------------------------------ router

// (value, index) of the largest entry of v[0..n), ties to the lower index; the whole warp takes part
__device__ __forceinline__ void warp_argmax(const float* v, int n, int lane, float& best, int& at) {
  best = -CUDART_INF_F;
  at = 0x7fffffff;
  for (int j = lane; j < n; j += 32) {
    const float x = v[j];
    if (x > best) { best = x; at = j; }      // ascending j: the first of equal entries stays
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oa = __shfl_xor_sync(0xffffffffu, at, o);
    if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
  }
}

// Router logits z[t][j] = Wr[j] . h[t] in fp32.  A block takes TOK tokens and RL_OB outputs; its eight warps share
// the k range (chunks of 128 dealt round-robin, 16-byte loads of the fp32 weight), so that even a single token's
// logits are a few loads deep; the warps' sums meet in shared memory in warp order.
constexpr int RL_WARPS = 8, RL_OB = 4;

template <typename T> struct Quad;
template <> struct Quad<float> {
  static __device__ __forceinline__ void load(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct Quad<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&v);
    const float2 a = __bfloat1622float2(hh[0]), b = __bfloat1622float2(hh[1]);
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
  }
};

template <typename T, int TOK, bool VEC>
__global__ void __launch_bounds__(RL_WARPS * 32)
moe_logits_kernel(const T* __restrict__ h, int ldh, const float* __restrict__ Wr, float* __restrict__ z, int tokens,
                  int d, int rows) {
  __shared__ float part[RL_WARPS][RL_OB * TOK];
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t0 = blockIdx.x * TOK;
  const int nt = min(TOK, tokens - t0);
  const int j0 = blockIdx.y * RL_OB;
  // rows beyond the last output or token stand in as the last one (their sums are never stored), so that no
  // load sits behind a branch and a whole iteration's loads are in flight together
  const float* wr[RL_OB];
#pragma unroll
  for (int o = 0; o < RL_OB; ++o) wr[o] = Wr + (size_t)min(j0 + o, rows - 1) * d;
  const T* hrow[TOK];
#pragma unroll
  for (int i = 0; i < TOK; ++i) hrow[i] = h + (size_t)(t0 + min(i, nt - 1)) * ldh;
  float acc[RL_OB][TOK];
#pragma unroll
  for (int o = 0; o < RL_OB; ++o)
#pragma unroll
    for (int i = 0; i < TOK; ++i) acc[o][i] = 0.f;
  pdl_wait();
  if (VEC) {
    for (int k = warp * 128 + lane * 4; k < d; k += RL_WARPS * 128) {
      float wv[RL_OB][4], hv[TOK][4];
#pragma unroll
      for (int o = 0; o < RL_OB; ++o) Quad<float>::load(wr[o] + k, wv[o]);
#pragma unroll
      for (int i = 0; i < TOK; ++i) Quad<T>::load(hrow[i] + k, hv[i]);
#pragma unroll
      for (int i = 0; i < TOK; ++i)
#pragma unroll
        for (int o = 0; o < RL_OB; ++o)
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[o][i] = fmaf(wv[o][c], hv[i][c], acc[o][i]);
    }
  } else {
    for (int k = warp * 32 + lane; k < d; k += RL_WARPS * 32) {
      float wv[RL_OB], hv[TOK];
#pragma unroll
      for (int o = 0; o < RL_OB; ++o) wv[o] = wr[o][k];
#pragma unroll
      for (int i = 0; i < TOK; ++i) hv[i] = to_float(hrow[i][k]);
#pragma unroll
      for (int i = 0; i < TOK; ++i)
#pragma unroll
        for (int o = 0; o < RL_OB; ++o) acc[o][i] = fmaf(wv[o], hv[i], acc[o][i]);
    }
  }
#pragma unroll
  for (int o = 0; o < RL_OB; ++o)
#pragma unroll
    for (int i = 0; i < TOK; ++i) {
      const float sum = warp_sum(acc[o][i]);
      if (lane == 0) part[warp][o * TOK + i] = sum;
    }
  __syncthreads();
  if (threadIdx.x < RL_OB * TOK) {
    const int o = threadIdx.x / TOK, i = threadIdx.x % TOK;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < RL_WARPS; ++w) sum += part[w][threadIdx.x];
    if (i < nt && j0 + o < rows) z[(size_t)(t0 + i) * rows + j0 + o] = sum;
  }
}

// The choice: a warp per token over its row of logits.
constexpr int RC_WARPS = 4;

// One token's choice by one warp; zt / ct / gt are the warp's scratch rows (rows, n and groups floats).
__device__ __forceinline__ void choose_token(const float* __restrict__ zg, const float* __restrict__ corr,
                                             const float* __restrict__ zbias, int* __restrict__ idx, float* __restrict__ wt, float* __restrict__ gate,
                                             int t, int n, int has_gate, int top, int groups, int keep,
                                             int sigmoid_scores, int renormalize, float* zt, float* ct, float* gt,
                                             int lane) {
  const int rows = n + (has_gate ? 1 : 0);
  for (int j = lane; j < rows; j += 32) zt[j] = zg[(size_t)t * rows + j] + (zbias != nullptr && j < n ? zbias[j] : 0.f);
  __syncwarp();
  if (has_gate && lane == 0) gate[t] = 1.f / (1.f + expf(-zt[n]));
  if (sigmoid_scores) {
    for (int j = lane; j < n; j += 32) zt[j] = 1.f / (1.f + expf(-zt[j]));
  } else {
    float m = -CUDART_INF_F;
    for (int j = lane; j < n; j += 32) m = fmaxf(m, zt[j]);
    m = warp_max(m);
    float sum = 0.f;
    for (int j = lane; j < n; j += 32) {
      const float e = expf(zt[j] - m);
      zt[j] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    for (int j = lane; j < n; j += 32) zt[j] = zt[j] / sum;
  }
  for (int j = lane; j < n; j += 32) ct[j] = zt[j] + (corr != nullptr ? corr[j] : 0.f);
  __syncwarp();
  if (keep < groups) {
    const int gsz = n / groups;
    for (int g = lane; g < groups; g += 32) {
      float m = -CUDART_INF_F;
      for (int j = 0; j < gsz; ++j) m = fmaxf(m, ct[g * gsz + j]);
      gt[g] = m;
    }
    __syncwarp();
    // a group that is found leaves the next rounds with a score of minus infinity (choice scores are finite);
    // the groups that still hold a finite score afterwards are the ones not kept, and lose their outputs
    for (int r = 0; r < keep; ++r) {
      float best;
      int at;
      warp_argmax(gt, groups, lane, best, at);
      __syncwarp();
      if (lane == 0 && at < groups) gt[at] = -CUDART_INF_F;
      __syncwarp();
    }
    for (int g = 0; g < groups; ++g) {
      if (gt[g] != -CUDART_INF_F)
        for (int j = lane; j < gsz; j += 32) ct[g * gsz + j] = -CUDART_INF_F;
    }
    __syncwarp();
  }
  float wsum = 0.f;
  for (int r = 0; r < top; ++r) {
    float best;
    int at;
    warp_argmax(ct, n, lane, best, at);
    if (at >= n) at = 0;                     // nothing left to choose (cannot happen for a checked configuration)
    const float wv = zt[at];
    wsum += wv;
    __syncwarp();
    if (lane == 0) {
      idx[(size_t)t * top + r] = at;
      wt[(size_t)t * top + r] = wv;
      ct[at] = -CUDART_INF_F;
    }
    __syncwarp();
  }
  if (renormalize)
    for (int r = lane; r < top; r += 32) wt[(size_t)t * top + r] /= wsum;
}

__global__ void __launch_bounds__(RC_WARPS * 32)
moe_choose_kernel(const float* __restrict__ zg, const float* __restrict__ corr, const float* __restrict__ zbias,
                  int* __restrict__ idx,
                  float* __restrict__ wt, float* __restrict__ gate, int tokens, int n, int has_gate, int top, int groups,
                  int keep, int sigmoid_scores, int renormalize) {
  extern __shared__ float rt_smem[];
  pdl_launch_dependents();
  const int rows = n + (has_gate ? 1 : 0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* zt = rt_smem + (size_t)warp * (rows + n + groups);      // scores
  const int t = blockIdx.x * RC_WARPS + warp;
  pdl_wait();
  if (t >= tokens) return;
  choose_token(zg, corr, zbias, idx, wt, gate, t, n, has_gate, top, groups, keep, sigmoid_scores, renormalize, zt, zt + rows,
               zt + rows + n, lane);
}

// -------------------------------------------------------------------------------------------- plan
constexpr int PLAN_THREADS = 1024;

// The whole block; count / cursor are n_experts ints of shared memory each, count zeroed (and a barrier passed).
__device__ __forceinline__ void plan_block(const int* __restrict__ idx, int pairs, int n_experts, int tile_rows,
                                           int* __restrict__ offsets, int* __restrict__ sorted_pair,
                                           int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                           int* __restrict__ n_tiles, int max_tiles, int* count, int* cursor) {
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = idx[i];
    if (e >= 0 && e < n_experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < n_experts; ++e) {
      offsets[e] = off;
      cursor[e] = off;
      for (int r = 0; r < count[e]; r += tile_rows) {
        if (nt < max_tiles) {
          tile_expert[nt] = e;
          tile_row0[nt] = off + r;
        }
        ++nt;
      }
      off += count[e];
    }
    offsets[n_experts] = off;
    *n_tiles = min(nt, max_tiles);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = idx[i];
    if (e >= 0 && e < n_experts) sorted_pair[atomicAdd(&cursor[e], 1)] = i;
  }
}

__global__ void __launch_bounds__(PLAN_THREADS)
moe_plan_kernel(const int* __restrict__ idx, int pairs, int n_experts, int tile_rows, int* __restrict__ offsets,
                int* __restrict__ sorted_pair, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                int* __restrict__ n_tiles, int max_tiles) {
  extern __shared__ int pl_smem[];
  int* count = pl_smem;                  // [n_experts]
  int* cursor = count + n_experts;       // [n_experts]
  pdl_launch_dependents();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  pdl_wait();
  plan_block(idx, pairs, n_experts, tile_rows, offsets, sorted_pair, tile_expert, tile_row0, n_tiles, max_tiles, count,
             cursor);
}

// Choice and plan of a step of few tokens in one launch: one block, a warp per token in turn, then the plan.
__global__ void __launch_bounds__(PLAN_THREADS)
moe_choose_plan_kernel(const float* __restrict__ zg, const float* __restrict__ corr,
                       const float* __restrict__ zbias, int* __restrict__ idx,
                       float* __restrict__ wt, float* __restrict__ gate, int tokens, int n, int has_gate, int top,
                       int groups, int keep, int sigmoid_scores, int renormalize, int n_experts, int tile_rows,
                       int* __restrict__ offsets, int* __restrict__ sorted_pair, int* __restrict__ tile_expert,
                       int* __restrict__ tile_row0, int* __restrict__ n_tiles, int max_tiles) {
  extern __shared__ float rt_smem[];
  pdl_launch_dependents();
  const int rows = n + (has_gate ? 1 : 0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  float* zt = rt_smem + (size_t)warp * (rows + n + groups);
  int* count = reinterpret_cast<int*>(rt_smem + (size_t)n_warps * (rows + n + groups));
  int* cursor = count + n_experts;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = 0;
  pdl_wait();
  for (int t = warp; t < tokens; t += n_warps) {
    choose_token(zg, corr, zbias, idx, wt, gate, t, n, has_gate, top, groups, keep, sigmoid_scores, renormalize, zt, zt + rows,
                 zt + rows + n, lane);
    __syncwarp();
  }
  __syncthreads();          // every choice is written (and the counts are zero) before anyone counts
  plan_block(idx, tokens * top, n_experts, tile_rows, offsets, sorted_pair, tile_expert, tile_row0, n_tiles, max_tiles,
             count, cursor);
}

// ------------------------------------------------------------------ grouped contraction: few rows
// Tiles of up to 8 rows of one expert; a warp per output column, lanes along k with 16-byte loads.
constexpr int FR_ROWS = 8, FR_WARPS = 8;

template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(hh[i]);
      o[2 * i] = f.x;
      o[2 * i + 1] = f.y;
    }
  }
};

struct GroupedArgs {
  const void* A;              // rows of K numbers
  long long lda;
  const int* a_gather;        // null: row r of A is sorted row r; else row a_gather[r] / a_div
  int a_div;
  const void* W;              // [experts][N][K]
  void* out;
  long long ldo;
  const int* o_scatter;       // null: sorted row r goes to row r of out; else to row o_scatter[r]
  const int* offsets;         // [experts + 1]
  const int* tile_expert;
  const int* tile_row0;
  const int* n_tiles;
  int N, K, act, out_f32;
};

template <typename T, bool VEC>
__global__ void __launch_bounds__(FR_WARPS * 32)
moe_gemm_few_kernel(GroupedArgs g) {
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= *g.n_tiles) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e = g.tile_expert[tile], r0 = g.tile_row0[tile];
  const int nr = min(FR_ROWS, g.offsets[e + 1] - r0);
  const T* arow[FR_ROWS];
#pragma unroll
  for (int i = 0; i < FR_ROWS; ++i) {
    const int r = r0 + min(i, nr - 1);
    const long long src = g.a_gather != nullptr ? g.a_gather[r] / g.a_div : r;
    arow[i] = (const T*)g.A + src * g.lda;
  }
  const int K = g.K;
  const T* Wexp = (const T*)g.W + (size_t)e * g.N * K;
  for (int n = blockIdx.x * FR_WARPS + warp; n < g.N; n += gridDim.x * FR_WARPS) {
    const T* wr = Wexp + (size_t)n * K;
    float acc[FR_ROWS];
#pragma unroll
    for (int i = 0; i < FR_ROWS; ++i) acc[i] = 0.f;
    if (VEC) {
      constexpr int V = Vec16<T>::N;
      for (int k = lane * V; k < K; k += 32 * V) {
        float wv[V];
        Vec16<T>::load(wr + k, wv);
#pragma unroll
        for (int i = 0; i < FR_ROWS; ++i) {
          if (i < nr) {
            float av[V];
            Vec16<T>::load(arow[i] + k, av);
#pragma unroll
            for (int j = 0; j < V; ++j) acc[i] = fmaf(wv[j], av[j], acc[i]);
          }
        }
      }
    } else {
      for (int k = lane; k < K; k += 32) {
        const float wv = to_float(wr[k]);
#pragma unroll
        for (int i = 0; i < FR_ROWS; ++i)
          if (i < nr) acc[i] = fmaf(wv, to_float(arow[i][k]), acc[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < FR_ROWS; ++i) {
      const float s = warp_sum(acc[i]);
      if (lane == 0 && i < nr) {
        const int r = r0 + i;
        const long long dst = (g.o_scatter != nullptr ? g.o_scatter[r] : r) * g.ldo + n;
        const float v = apply_act(s, g.act);
        if (g.out_f32) ((float*)g.out)[dst] = v;
        else ((T*)g.out)[dst] = from_float<T>(v);
      }
    }
  }
}

// ----------------------------------------------------------------- grouped contraction: many rows
// 64 x 64 tiles on the fp32 pipes, each output one running sum over k in index order.
constexpr int GB = 64, GK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
moe_gemm_tiles_kernel(GroupedArgs g) {
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= *g.n_tiles) return;
  __shared__ float As[GK][GB + 4];
  __shared__ float Ws[GK][GB + 4];
  __shared__ long long a_src[GB];
  __shared__ long long o_dst[GB];
  const int tid = threadIdx.x;
  const int e = g.tile_expert[tile], r0 = g.tile_row0[tile];
  const int nr = min(GB, g.offsets[e + 1] - r0);
  const int n0 = blockIdx.x * GB;
  const int K = g.K, N = g.N;
  if (tid < GB) {
    const int r = r0 + min(tid, nr - 1);
    a_src[tid] = (g.a_gather != nullptr ? g.a_gather[r] / g.a_div : r) * g.lda;
    o_dst[tid] = (long long)(g.o_scatter != nullptr ? g.o_scatter[r] : r) * g.ldo;
  }
  __syncthreads();
  const T* A = (const T*)g.A;
  const T* Wexp = (const T*)g.W + (size_t)e * N * K;
  const int ty = tid / 16, tx = tid % 16;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += GK) {
    {
      const T* ap = A + a_src[lrow] + k0 + lk;
#pragma unroll
      for (int j = 0; j < 4; ++j) As[lk + j][lrow] = (lrow < nr && k0 + lk + j < K) ? to_float(ap[j]) : 0.f;
      const int gn = n0 + lrow;
      const T* wp = Wexp + (size_t)gn * K + k0 + lk;
#pragma unroll
      for (int j = 0; j < 4; ++j) Ws[lk + j][lrow] = (gn < N && k0 + lk + j < K) ? to_float(wp[j]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lr = ty * 4 + i;
    if (lr >= nr) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      const float v = apply_act(acc[i][j], g.act);
      if (g.out_f32) ((float*)g.out)[o_dst[lr] + gn] = v;
      else ((T*)g.out)[o_dst[lr] + gn] = from_float<T>(v);
    }
  }
}

// ----------------------------------------------------------------------------------------- combine
// A thread per token and four neighbouring channels (16-byte accesses where rows allow); P is the type of the
// experts' results (fp32 or the run's type).
template <typename T, typename P, bool VEC>
__global__ void __launch_bounds__(256)
moe_combine_kernel(float* __restrict__ y, const P* __restrict__ pair_out, const T* __restrict__ h, int ldh,
                   const int* __restrict__ idx, const float* __restrict__ wt, const float* __restrict__ shared,
                   const float* __restrict__ gate, int tokens, int d, int top, int n_experts) {
  pdl_launch_dependents();
  constexpr int W = VEC ? 4 : 1;
  const int per_row = (d + W - 1) / W;
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_wait();
  if (item >= (long long)tokens * per_row) return;
  const int t = (int)(item / per_row), i = (int)(item - (long long)t * per_row) * W;
  float acc[W];
#pragma unroll
  for (int c = 0; c < W; ++c) acc[c] = 0.f;
  for (int k = 0; k < top; ++k) {
    const int e = idx[(size_t)t * top + k];
    const float wk = wt != nullptr ? wt[(size_t)t * top + k] : 1.f;
    float v[W];
    if (e < n_experts) {
      const P* src = pair_out + ((size_t)t * top + k) * d + i;
      if (VEC) Quad<P>::load(src, v); else v[0] = to_float(src[0]);
    } else {
      const T* src = h + (size_t)t * ldh + i;
      if (VEC) Quad<T>::load(src, v); else v[0] = to_float(src[0]);
    }
#pragma unroll
    for (int c = 0; c < W; ++c) acc[c] = fmaf(wk, v[c], acc[c]);
  }
  if (shared != nullptr) {
    const float gt = gate != nullptr ? gate[t] : 1.f;
    float v[W];
    if (VEC) Quad<float>::load(shared + (size_t)t * d + i, v); else v[0] = shared[(size_t)t * d + i];
#pragma unroll
    for (int c = 0; c < W; ++c) acc[c] = fmaf(gt, v[c], acc[c]);
  }
  float* yr = y + (size_t)t * d + i;
  if (VEC) {
    float4 o = *reinterpret_cast<float4*>(yr);
    o.x += acc[0]; o.y += acc[1]; o.z += acc[2]; o.w += acc[3];
    *reinterpret_cast<float4*>(yr) = o;
  } else {
    yr[0] += acc[0];
  }
}

// ------------------------------------------------------------------------------ weights on the input
// For experts whose weight multiplies their INPUT (y = sum_k expert_k(w_k h), which is not w_k expert_k(h) once
// an expert is not linear): one row per (token, choice) pair, rows[t * top + k] = w[t][k] * h[t] in the run's
// type (the product in fp32); the combine then adds the experts' results as they are (no weights).
template <typename T>
__global__ void moe_scale_rows_kernel(const T* h, int ldh, const float* wt, T* rows, int d, int top) {
  pdl_launch_dependents();
  const int p = blockIdx.x;
  pdl_wait();
  const float w = wt[p];
  const T* src = h + (size_t)(p / top) * ldh;
  T* dst = rows + (size_t)p * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = from_float<T>(w * to_float(src[i]));
}

template <typename T, typename P>
static void launch_combine(float* y, const void* pair_out, const void* h, int ldh, const int* idx, const float* wt,
                           const float* shared, const float* gate, int tokens, int d, int top, int n_experts,
                           cudaStream_t stream) {
  const bool vec = d % 4 == 0 && ldh % 4 == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)pair_out % 16) == 0 &&
                   ((uintptr_t)h % 16) == 0 && ((uintptr_t)shared % 16) == 0;
  const long long items = (long long)tokens * (vec ? d / 4 : d);
  dim3 grid((unsigned)((items + 255) / 256)), block(256);
  if (vec)
    launch_kernel(moe_combine_kernel<T, P, true>, grid, block, 0, stream, y, (const P*)pair_out, (const T*)h, ldh, idx,
                  wt, shared, gate, tokens, d, top, n_experts);
  else
    launch_kernel(moe_combine_kernel<T, P, false>, grid, block, 0, stream, y, (const P*)pair_out, (const T*)h, ldh, idx,
                  wt, shared, gate, tokens, d, top, n_experts);
}

}  // namespace dlgo

using namespace dlgo;

template <typename T>
static void launch_logits(const void* h, int ldh, const float* Wr, float* z, int tokens, int d, int rows,
                          cudaStream_t stream) {
  const bool vec = d % 4 == 0 && ldh % 4 == 0 && ((uintptr_t)h % 16) == 0 && ((uintptr_t)Wr % 16) == 0;
  const int by = (rows + RL_OB - 1) / RL_OB;
  dim3 block(RL_WARPS * 32);
  if (tokens <= 64) {
    dim3 grid((tokens + 7) / 8, by);
    if (vec) launch_kernel(moe_logits_kernel<T, 8, true>, grid, block, 0, stream, (const T*)h, ldh, Wr, z, tokens, d, rows);
    else launch_kernel(moe_logits_kernel<T, 8, false>, grid, block, 0, stream, (const T*)h, ldh, Wr, z, tokens, d, rows);
  } else {
    dim3 grid((tokens + 15) / 16, by);
    if (vec) launch_kernel(moe_logits_kernel<T, 16, true>, grid, block, 0, stream, (const T*)h, ldh, Wr, z, tokens, d, rows);
    else launch_kernel(moe_logits_kernel<T, 16, false>, grid, block, 0, stream, (const T*)h, ldh, Wr, z, tokens, d, rows);
  }
}

// Two launches: the logits z [tokens, n (+ 1)] (scratch, fp32), then the choice.  With plan_experts > 0 and few
// tokens the second launch also makes the plan (as dlgo_moe_plan would from idx); *fused says whether it did.
DLGO_EXPORT int dlgo_moe_router(const void* h, int dtype, int ldh, const float* Wr, const float* corr,
                                const float* zbias, float* z, int* idx,
                                float* wt, float* gate, int tokens, int d, int n, int has_gate, int top, int groups,
                                int keep, int sigmoid_scores, int renormalize, int plan_experts, int tile_rows,
                                int* offsets, int* sorted_pair, int* tile_expert, int* tile_row0, int* n_tiles,
                                int max_tiles, int* fused, cudaStream_t stream) {
  if (fused != nullptr) *fused = 0;
  if (tokens <= 0) return DLGO_OK;
  if (n <= 0 || top <= 0 || top > n || groups <= 0 || n % groups || keep <= 0 || keep > groups || d <= 0)
    return DLGO_ERR_SIZE;
  const int rows = n + (has_gate ? 1 : 0);
  const size_t smem = sizeof(float) * RC_WARPS * ((size_t)rows + n + groups);
  if (smem > 48 * 1024) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32) launch_logits<float>(h, ldh, Wr, z, tokens, d, rows, stream);
  else if (dtype == DLGO_BF16) launch_logits<__nv_bfloat16>(h, ldh, Wr, z, tokens, d, rows, stream);
  else return DLGO_ERR_DTYPE;
  int st = launch_status();
  if (st != DLGO_OK) return st;
  if (plan_experts > 0 && fused != nullptr && tokens <= 64) {
    const int warps = tokens <= 8 ? 8 : (tokens <= 16 ? 16 : 32);
    const size_t both = sizeof(float) * warps * ((size_t)rows + n + groups) + sizeof(int) * 2 * (size_t)plan_experts;
    const int pairs = tokens * top;
    if (both <= 48 * 1024 && tile_rows > 0 && max_tiles >= (pairs + tile_rows - 1) / tile_rows + plan_experts) {
      launch_kernel(moe_choose_plan_kernel, dim3(1), dim3(warps * 32), both, stream, (const float*)z, corr, zbias, idx, wt, gate,
                    tokens, n, has_gate, top, groups, keep, sigmoid_scores, renormalize, plan_experts, tile_rows, offsets,
                    sorted_pair, tile_expert, tile_row0, n_tiles, max_tiles);
      *fused = 1;
      return launch_status();
    }
  }
  launch_kernel(moe_choose_kernel, dim3((tokens + RC_WARPS - 1) / RC_WARPS), dim3(RC_WARPS * 32), smem, stream,
                (const float*)z, corr, zbias, idx, wt, gate, tokens, n, has_gate, top, groups, keep, sigmoid_scores, renormalize);
  return launch_status();
}

DLGO_EXPORT int dlgo_moe_plan(const int* idx, int pairs, int n_experts, int tile_rows, int* offsets, int* sorted_pair,
                              int* tile_expert, int* tile_row0, int* n_tiles, int max_tiles, cudaStream_t stream) {
  if (pairs <= 0 || n_experts <= 0) return DLGO_ERR_SIZE;
  if (tile_rows <= 0 || max_tiles < (pairs + tile_rows - 1) / tile_rows + n_experts) return DLGO_ERR_SIZE;
  const size_t smem = sizeof(int) * 2 * (size_t)n_experts;
  if (smem > 48 * 1024) return DLGO_ERR_SIZE;
  launch_kernel(moe_plan_kernel, dim3(1), dim3(PLAN_THREADS), smem, stream, idx, pairs, n_experts, tile_rows, offsets,
                sorted_pair, tile_expert, tile_row0, n_tiles, max_tiles);
  return launch_status();
}

// kind 0: tiles of 8 rows (few rows per expert); kind 1: 64 x 64 tiles.  `max_tiles` sizes the grid.
DLGO_EXPORT int dlgo_moe_gemm(int kind, int dtype, const void* A, long long lda, const int* a_gather, int a_div,
                              const void* W, void* out, long long ldo, const int* o_scatter, const int* offsets,
                              const int* tile_expert, const int* tile_row0, const int* n_tiles, int max_tiles, int N,
                              int K, int act, int out_f32, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0 || K <= 0 || max_tiles > 65535 || a_div <= 0) return DLGO_ERR_SIZE;
  GroupedArgs g{A, lda, a_gather, a_div, W, out, ldo, o_scatter, offsets, tile_expert, tile_row0, n_tiles, N, K, act, out_f32};
  const size_t esz = dtype == DLGO_F32 ? 4 : 2;
  if (dtype != DLGO_F32 && dtype != DLGO_BF16) return DLGO_ERR_DTYPE;
  if (kind == 0) {
    const int vec = 16 / (int)esz;
    const bool can_vec = K % vec == 0 && lda % vec == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0;
    // columns per block: as many blocks along N as keep every SM busy with few tiles
    int bx = (N + FR_WARPS - 1) / FR_WARPS;
    dim3 grid(bx, max_tiles), block(FR_WARPS * 32);
    if (dtype == DLGO_F32) {
      if (can_vec) launch_kernel(moe_gemm_few_kernel<float, true>, grid, block, 0, stream, g);
      else launch_kernel(moe_gemm_few_kernel<float, false>, grid, block, 0, stream, g);
    } else {
      if (can_vec) launch_kernel(moe_gemm_few_kernel<__nv_bfloat16, true>, grid, block, 0, stream, g);
      else launch_kernel(moe_gemm_few_kernel<__nv_bfloat16, false>, grid, block, 0, stream, g);
    }
  } else if (kind == 1) {
    dim3 grid((N + GB - 1) / GB, max_tiles), block(256);
    if (dtype == DLGO_F32) launch_kernel(moe_gemm_tiles_kernel<float>, grid, block, 0, stream, g);
    else launch_kernel(moe_gemm_tiles_kernel<__nv_bfloat16>, grid, block, 0, stream, g);
  } else {
    return DLGO_ERR_SIZE;
  }
  return launch_status();
}

// pair_out: the experts' results [tokens * top, d], fp32 (pair_f32) or of h's type
DLGO_EXPORT int dlgo_moe_scale_rows(const void* h, int dtype, int ldh, const float* wt, void* rows, int pairs, int d,
                                    int top, cudaStream_t stream) {
  if (pairs <= 0) return DLGO_OK;
  if (d <= 0 || top <= 0) return DLGO_ERR_SIZE;
  const int threads = d >= 1024 ? 256 : 128;
  if (dtype == DLGO_F32)
    launch_kernel(moe_scale_rows_kernel<float>, dim3(pairs), dim3(threads), 0, stream, (const float*)h, ldh, wt,
                  (float*)rows, d, top);
  else if (dtype == DLGO_BF16)
    launch_kernel(moe_scale_rows_kernel<__nv_bfloat16>, dim3(pairs), dim3(threads), 0, stream, (const __nv_bfloat16*)h,
                  ldh, wt, (__nv_bfloat16*)rows, d, top);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

DLGO_EXPORT int dlgo_moe_combine(float* y, const void* pair_out, int pair_f32, const void* h, int dtype, int ldh,
                                 const int* idx, const float* wt, const float* shared, const float* gate, int tokens,
                                 int d, int top, int n_experts, cudaStream_t stream) {
  if (tokens <= 0) return DLGO_OK;
  if (d <= 0 || top <= 0) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32)
    launch_combine<float, float>(y, pair_out, h, ldh, idx, wt, shared, gate, tokens, d, top, n_experts, stream);
  else if (dtype == DLGO_BF16 && pair_f32)
    launch_combine<__nv_bfloat16, float>(y, pair_out, h, ldh, idx, wt, shared, gate, tokens, d, top, n_experts, stream);
  else if (dtype == DLGO_BF16)
    launch_combine<__nv_bfloat16, __nv_bfloat16>(y, pair_out, h, ldh, idx, wt, shared, gate, tokens, d, top, n_experts,
                                                 stream);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}
