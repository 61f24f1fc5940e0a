// Attention over a cache of latents (one vector of `rank` numbers per position, shared by all heads).
//
// Per position the cache holds c = rms(Wd h) * g.  A head's keys and values are k = Wk c and v = Wv c, so
//   score(i, j) = q_i . (Wk c_j) * scale = (Wk^T q_i) . c_j * scale
//   out_i       = Wv (sum_j p_ij c_j)
// and neither keys nor values are ever materialised: the query is carried into the latent space once, the
// softmax runs over the latents themselves, and the weighted latent is carried out through Wv at the end.
// Causal; `window` > 0 keeps keys with 0 <= i - j < window; `sink` (one number per head) adds exp(sink) to the
// softmax's denominator and nothing else.  No positions are encoded.
//
// latent_norm_append: the RMS norms of the down-projections (fp32), the kv latent appended to the paged
// cache, the query latent (if the queries go through one) handed on in the activation type.
// latent_attention:   one block per (token, head), all arithmetic in fp32; T is the type of the cache, the
//                     weights and the output.  Keys are spread over the block's warps in a fixed pattern, so a
//                     token's result does not depend on what else is in the batch.
#include "common.cuh"

namespace dlgo {

template <typename T>
__global__ void latent_norm_append_kernel(const float* __restrict__ proj, int ld, int kv_off, int kv_rank,
                                          const float* __restrict__ w_kv, int q_off, int q_rank,
                                          const float* __restrict__ w_q, T* __restrict__ cq, float eps,
                                          const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                                          const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                                          int max_pages, T* __restrict__ pages, int page_size, int write_cache) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  __shared__ float scale_s;
  const int t = blockIdx.x;
  const bool is_q = blockIdx.y == 1;
  const int n = is_q ? q_rank : kv_rank;
  const float* w = is_q ? w_q : w_kv;
  T* dst = nullptr;
  if (is_q) {
    dst = cq + (size_t)t * q_rank;
  } else if (write_cache) {
    const int pos = token_pos[t];
    const int slot = seq_slot[token_seq[t]];
    const int page = page_table[(size_t)slot * max_pages + pos / page_size];
    if (page >= 0) dst = pages + ((size_t)page * page_size + pos % page_size) * kv_rank;
  }
  pdl_wait();
  if (dst == nullptr) return;
  const float* x = proj + (size_t)t * ld + (is_q ? q_off : kv_off);
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) scale_s = 1.0f / sqrtf(ss / (float)n + eps);
  __syncthreads();
  const float sc = scale_s;
  for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = from_float<T>(x[i] * sc * w[i]);
}

// The same for latents that carry a rotated key part: the down-projection has kv_rank + rope numbers; the first
// kv_rank are normed (times w_kv) as above, the last `rope` are one key part shared by all heads, which turns with
// the position (entries 2i and 2i + 1 by the angle pos * freq[i], cosine and sine times `amplitude`) and is kept
// behind the latent in the same cache row ([.., page, kv_rank + rope]).  Queries q [T, H, dq] (fp32, inside
// proj at q_off) turn in place in their last `rope` numbers of every head.  blockIdx.y: 0 the cache row, 1 the
// queries.  Angles are float(pos) * freq in fp32.
template <typename T>
__global__ void latent_rope_append_kernel(float* proj, int ld, int kv_off, int kv_rank, const float* __restrict__ w_kv,
                                          int q_off, int H, int dq, int rope, const float* __restrict__ freq,
                                          float amplitude, float eps, const int* __restrict__ token_pos,
                                          const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                          const int* __restrict__ page_table, int max_pages, T* pages, int page_size,
                                          int write_cache) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  __shared__ float scale_s;
  const int t = blockIdx.x;
  const int pos = token_pos[t];
  const int half = rope / 2;
  if (blockIdx.y == 1) {
    pdl_wait();
    float* q = proj + (size_t)t * ld + q_off;
    for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
      const int h = idx / half, i = idx - h * half;
      float* pair = q + (size_t)h * dq + (dq - rope) + 2 * i;
      float sn, cs;
      sincosf((float)pos * freq[i], &sn, &cs);
      sn *= amplitude;
      cs *= amplitude;
      const float u = pair[0], v = pair[1];
      pair[0] = u * cs - v * sn;
      pair[1] = v * cs + u * sn;
    }
    return;
  }
  T* dst = nullptr;
  if (write_cache) {
    const int slot = seq_slot[token_seq[t]];
    const int page = page_table[(size_t)slot * max_pages + pos / page_size];
    if (page >= 0) dst = pages + ((size_t)page * page_size + pos % page_size) * (kv_rank + rope);
  }
  pdl_wait();
  if (dst == nullptr) return;
  const float* x = proj + (size_t)t * ld + kv_off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) scale_s = 1.0f / sqrtf(ss / (float)kv_rank + eps);
  __syncthreads();
  const float sc = scale_s;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) dst[i] = from_float<T>(x[i] * sc * w_kv[i]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * freq[i], &sn, &cs);
    sn *= amplitude;
    cs *= amplitude;
    const float u = x[kv_rank + 2 * i], v = x[kv_rank + 2 * i + 1];
    dst[kv_rank + 2 * i] = from_float<T>(u * cs - v * sn);
    dst[kv_rank + 2 * i + 1] = from_float<T>(v * cs + u * sn);
  }
}

// Latents of the pages a prompt step attends, gathered into rows [n_tmp * page_size, rank] (row = temporary page
// * page_size + place in the page) for the contraction that makes the step's keys and values.  `tmp_pages`
// [n_tmp, 3]: (sequence of the step, its page index, rows of the page that are written); other rows are zero.
constexpr int GATHER_PARTS = 8;     // blocks that share a page

template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ pages, const int* __restrict__ page_table, int max_pages,
                                     int page_size, const int* __restrict__ tmp_pages,
                                     const int* __restrict__ seq_slot, T* __restrict__ out, int rank) {
  pdl_launch_dependents();
  const int tp = blockIdx.x;
  const int seq = tmp_pages[tp * 3], lp = tmp_pages[tp * 3 + 1], valid = tmp_pages[tp * 3 + 2];
  const int page = page_table[(size_t)seq_slot[seq] * max_pages + lp];
  pdl_wait();
  const T* src = pages + (size_t)(page < 0 ? 0 : page) * page_size * rank;
  T* dst = out + (size_t)tp * page_size * rank;
  const int total = page_size * rank, n_valid = page < 0 ? 0 : valid * rank;
  const int per = (total + GATHER_PARTS - 1) / GATHER_PARTS;
  const int lo = blockIdx.y * per, hi = min(total, lo + per);
  constexpr int V = 16 / (int)sizeof(T);                         // elements of a 16-byte piece
  if ((rank % V) == 0 && (per % V) == 0 && ((uintptr_t)pages & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    // written rows end at a multiple of `rank`, so a 16-byte piece is wholly written or wholly not
    for (int i = lo + threadIdx.x * V; i < hi; i += blockDim.x * V)
      *reinterpret_cast<uint4*>(dst + i) = i < n_valid ? __ldg(reinterpret_cast<const uint4*>(src + i))
                                                        : make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) dst[i] = i < n_valid ? src[i] : from_float<T>(0.f);
}

__device__ __forceinline__ float2 load_pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// a pair of neighbouring elements; `vec`: the pair is 2-element aligned and wholly inside the row
template <typename T>
__device__ __forceinline__ float2 load_pair_any(const T* row, int r, int rank, bool vec) {
  if (vec) return load_pair(row + r);
  return make_float2(to_float(row[r]), r + 1 < rank ? to_float(row[r + 1]) : 0.f);
}

constexpr int LA_WARPS = 8;

// NP: pairs of latent dimensions a lane holds (rank <= 64 * NP, rank even)
template <typename T, int NP>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(const void* __restrict__ q, int q_is_f32, int ldq, const T* __restrict__ w_k,
                        const T* __restrict__ w_v, const float* __restrict__ sink, const T* __restrict__ pages,
                        const int* __restrict__ page_table, int max_pages, int page_size,
                        const int* __restrict__ seq_slot, const int* __restrict__ token_seq,
                        const int* __restrict__ token_pos, T* __restrict__ out, int ldo, int dk, int dv, int rank,
                        float scale, int window) {
  pdl_launch_dependents();
  extern __shared__ float smem[];
  float* s_q = smem;                         // [dk] the head's query
  float* s_lat = s_q + dk;                   // [rank] the query in latent space, later the weighted latent
  float* s_acc = s_lat + rank;               // [LA_WARPS][rank]
  __shared__ float s_m[LA_WARPS], s_l[LA_WARPS];
  const int t = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = token_pos[t];
  const int slot = seq_slot[token_seq[t]];
  const int* table = page_table + (size_t)slot * max_pages;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const bool vec = (rank & 1) == 0;          // rows start on a pair's boundary (the bases are 16-byte aligned)
  pdl_wait();
  for (int i = threadIdx.x; i < dk; i += blockDim.x)
    s_q[i] = q_is_f32 ? reinterpret_cast<const float*>(q)[(size_t)t * ldq + h * dk + i]
                      : to_float(reinterpret_cast<const __nv_bfloat16*>(q)[(size_t)t * ldq + h * dk + i]);
  __syncthreads();
  // the query in latent space: (Wk_h)^T q
  const T* wk = w_k + (size_t)h * dk * rank;
  for (int r = threadIdx.x; r < rank; r += blockDim.x) {
    float a = 0.f;
    for (int i = 0; i < dk; ++i) a = fmaf(s_q[i], to_float(wk[(size_t)i * rank + r]), a);
    s_lat[r] = a;
  }
  __syncthreads();
  float2 ql[NP], acc[NP];
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int r = (i * 32 + lane) * 2;
    ql[i] = r < rank ? make_float2(s_lat[r], r + 1 < rank ? s_lat[r + 1] : 0.f) : make_float2(0.f, 0.f);
    acc[i] = make_float2(0.f, 0.f);
  }
  float m = -INFINITY, l = 0.f;
  for (int j = lo + warp; j <= pos; j += LA_WARPS) {
    const int page = table[j / page_size];
    const T* c = pages + ((size_t)page * page_size + j % page_size) * rank;
    float2 cv[NP];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      const int r = (i * 32 + lane) * 2;
      cv[i] = r < rank ? load_pair_any(c, r, rank, vec) : make_float2(0.f, 0.f);
      s = fmaf(ql[i].x, cv[i].x, s);
      s = fmaf(ql[i].y, cv[i].y, s);
    }
    s = warp_sum(s) * scale;
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);        // 0 for the first key (m = -inf)
    const float p = expf(s - m_new);
    l = fmaf(l, corr, p);
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      acc[i].x = fmaf(acc[i].x, corr, p * cv[i].x);
      acc[i].y = fmaf(acc[i].y, corr, p * cv[i].y);
    }
    m = m_new;
  }
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int r = (i * 32 + lane) * 2;
    if (r < rank) s_acc[warp * rank + r] = acc[i].x;
    if (r + 1 < rank) s_acc[warp * rank + r + 1] = acc[i].y;
  }
  __syncthreads();
  // the warps' parts meet in warp order; the sink joins the denominator only
  const float sk = sink ? sink[h] : -INFINITY;
  float M = sk;
  for (int w = 0; w < LA_WARPS; ++w) M = fmaxf(M, s_m[w]);
  float L = sink ? expf(sk - M) : 0.f;
  float f[LA_WARPS];
#pragma unroll
  for (int w = 0; w < LA_WARPS; ++w) {
    f[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - M);
    L = fmaf(s_l[w], f[w], L);
  }
  const float inv = 1.0f / L;
  for (int r = threadIdx.x; r < rank; r += blockDim.x) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < LA_WARPS; ++w) a = fmaf(s_acc[w * rank + r], f[w], a);
    s_lat[r] = a * inv;
  }
  __syncthreads();
  // out through Wv_h: a warp per output column
  const T* wv = w_v + (size_t)h * dv * rank;
  for (int e = warp; e < dv; e += LA_WARPS) {
    const T* row = wv + (size_t)e * rank;
    float a = 0.f;
    for (int r = lane * 2; r < rank; r += 64) {
      const float2 wv2 = load_pair_any(row, r, rank, vec);
      a = fmaf(wv2.x, s_lat[r], a);
      if (r + 1 < rank) a = fmaf(wv2.y, s_lat[r + 1], a);
    }
    a = warp_sum(a);
    if (lane == 0) out[(size_t)t * ldo + h * dv + e] = from_float<T>(a);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Few tokens (decoding): three launches, each with enough blocks for the whole GPU.
//   absorb   q~[t, h, :] = (Wk_h)^T q[t, h, :]: a block per (head, 32 latent columns), its warps sharing the rows, reads its part of Wk
//            once for all tokens of the step
//   partial  a block per (token, head, slice of the visible keys): online softmax over the latents in fp32;
//            keys go round the block's warps, four in flight per warp.  Leaves (max, sum, weighted latent)
//   out      a block per (head, 8 value columns): the slices of a token meet in slice order, the sink joins the
//            denominator, and the weighted latent goes through its rows of Wv_h
constexpr int AB_TOKENS = 8;    // tokens whose sums a thread of `absorb` keeps at a time

constexpr int AB_COLS = 32;     // latent columns of a block (a lane each); its four warps share the rows of Wk_h

template <typename T>
__global__ void __launch_bounds__(128)
latent_absorb_kernel(const void* __restrict__ q, int q_is_f32, int ldq, const T* __restrict__ w_k,
                     float* __restrict__ q_lat, int n_tokens, int H, int dk, int rank) {
  pdl_launch_dependents();
  extern __shared__ float s_q[];                                // [AB_TOKENS][dk], then [4][AB_TOKENS][AB_COLS]
  float* s_part = s_q + AB_TOKENS * dk;
  const int h = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = blockIdx.y * AB_COLS + lane;
  const int t0 = blockIdx.z * AB_TOKENS;
  const int nt = min(AB_TOKENS, n_tokens - t0);
  // this warp's rows of Wk_h: weights, fetched (16 in flight) before the wait for the queries
  const int rows_per = (dk + 3) / 4;
  const int i0 = warp * rows_per, i1 = min(dk, i0 + rows_per);
  const T* wk = w_k + (size_t)h * dk * rank + (r < rank ? r : 0);
  float acc[AB_TOKENS];
#pragma unroll
  for (int t = 0; t < AB_TOKENS; ++t) acc[t] = 0.f;
  pdl_wait();
  for (int i = threadIdx.x; i < nt * dk; i += 128) {
    const int t = t0 + i / dk, c = h * dk + i % dk;
    s_q[i] = q_is_f32 ? reinterpret_cast<const float*>(q)[(size_t)t * ldq + c]
                      : to_float(reinterpret_cast<const __nv_bfloat16*>(q)[(size_t)t * ldq + c]);
  }
  __syncthreads();
  for (int ib = i0; ib < i1; ib += 16) {
    float w[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) w[k] = (ib + k < i1) ? to_float(wk[(size_t)(ib + k) * rank]) : 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      if (ib + k < i1) {
#pragma unroll
        for (int t = 0; t < AB_TOKENS; ++t) acc[t] = fmaf(s_q[t * dk + ib + k], w[k], acc[t]);   // (rows of absent tokens are unused)
      }
    }
  }
#pragma unroll
  for (int t = 0; t < AB_TOKENS; ++t) s_part[(warp * AB_TOKENS + t) * AB_COLS + lane] = acc[t];
  __syncthreads();
  // the four warps' sums meet in warp order; warp w writes tokens w, w + 4
  for (int t = warp; t < nt; t += 4) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) a += s_part[(w * AB_TOKENS + t) * AB_COLS + lane];
    if (r < rank) q_lat[((size_t)(t0 + t) * H + h) * rank + r] = a;
  }
}

constexpr int LP_WARPS = 4;
constexpr int LP_UNROLL = 4;

// 16 bytes of a latent row as floats: V = 8 bfloat16 or 4 float
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int V = 4;
  __device__ static __forceinline__ uint4 raw(const float* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
  __device__ static __forceinline__ void unpack(const uint4& u, float* o) {
    o[0] = __uint_as_float(u.x); o[1] = __uint_as_float(u.y); o[2] = __uint_as_float(u.z); o[3] = __uint_as_float(u.w);
  }
  __device__ static __forceinline__ void load(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int V = 8;
  __device__ static __forceinline__ uint4 raw(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
  __device__ static __forceinline__ void unpack(const uint4& u, float* o) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      o[2 * k] = f.x; o[2 * k + 1] = f.y;
    }
  }
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float* o) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      o[2 * k] = f.x; o[2 * k + 1] = f.y;
    }
  }
};

// parts [T, H, S, rank + 2]: (max, sum, weighted latent) of each slice.  A lane holds CH pieces of 16 bytes of a
// latent row (rank <= 32 * CH * V, rank a multiple of V); the page numbers and then the rows of LP_UNROLL keys are
// fetched together before any of them is used.
template <typename T, int CH>
__global__ void __launch_bounds__(LP_WARPS * 32)
latent_partial_kernel(const float* __restrict__ q_lat, const T* __restrict__ pages, const int* __restrict__ page_table,
                      int max_pages, int page_size, const int* __restrict__ seq_slot,
                      const int* __restrict__ token_seq, const int* __restrict__ token_pos, float* __restrict__ parts,
                      int H, int rank, int n_slices, float scale, int window) {
  constexpr int V = Vec16<T>::V;
  pdl_launch_dependents();
  extern __shared__ float s_acc[];                              // [LP_WARPS][rank]
  __shared__ float s_m[LP_WARPS], s_l[LP_WARPS];
  const int t = blockIdx.x, h = blockIdx.y, slice = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = token_pos[t];
  const int* table = page_table + (size_t)seq_slot[token_seq[t]] * max_pages;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int per = (pos - lo + n_slices) / n_slices;             // keys of a slice (the last may have fewer)
  const int j0 = lo + slice * per, j1 = min(pos + 1, j0 + per);
  pdl_wait();
  const float* ql_g = q_lat + ((size_t)t * H + h) * rank;
  float ql[CH][V], acc[CH][V];
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int r = (i * 32 + lane) * V;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      ql[i][k] = r < rank ? ql_g[r + k] : 0.f;
      acc[i][k] = 0.f;
    }
  }
  float m = -INFINITY, l = 0.f;
  // page numbers run one group ahead of the rows: a group costs one round trip to memory, not two
  int page_next[LP_UNROLL];
#pragma unroll
  for (int u = 0; u < LP_UNROLL; ++u) {
    const int j = j0 + warp * LP_UNROLL + u;
    page_next[u] = j < j1 ? table[j / page_size] : 0;
  }
  for (int jb = j0 + warp * LP_UNROLL; jb < j1; jb += LP_WARPS * LP_UNROLL) {
    int page[LP_UNROLL];
#pragma unroll
    for (int u = 0; u < LP_UNROLL; ++u) {
      page[u] = page_next[u];
      const int jn = jb + LP_WARPS * LP_UNROLL + u;
      page_next[u] = jn < j1 ? table[jn / page_size] : 0;
    }
    // Every fetch of the group is issued before any of them is used: no branch stands between them.  A key
    // beyond the slice's end stands in as the slice's last key (written, finite) and gets weight zero below;
    // a lane beyond the rank reads the row's start against a zero query.
    uint4 raw[LP_UNROLL][CH];
#pragma unroll
    for (int u = 0; u < LP_UNROLL; ++u) {
      const bool in = jb + u < j1;
      const int j = in ? jb + u : j1 - 1;
      const int pg = in ? page[u] : table[j / page_size];
      const T* row = pages + ((size_t)pg * page_size + j % page_size) * rank;
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int r = (i * 32 + lane) * V;
        raw[u][i] = Vec16<T>::raw(row + (r < rank ? r : 0));
      }
    }
    float cv[LP_UNROLL][CH][V];
#pragma unroll
    for (int u = 0; u < LP_UNROLL; ++u)
#pragma unroll
      for (int i = 0; i < CH; ++i) Vec16<T>::unpack(raw[u][i], cv[u][i]);
    float sc[LP_UNROLL];
#pragma unroll
    for (int u = 0; u < LP_UNROLL; ++u) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < CH; ++i)
#pragma unroll
        for (int k = 0; k < V; ++k) s = fmaf(ql[i][k], cv[u][i][k], s);
      sc[u] = (jb + u < j1) ? warp_sum(s) * scale : -INFINITY;
    }
    float m_new = m;
#pragma unroll
    for (int u = 0; u < LP_UNROLL; ++u) m_new = fmaxf(m_new, sc[u]);
    const float corr = expf(m - m_new);                         // (the first key of a group is always there)
    l *= corr;
#pragma unroll
    for (int i = 0; i < CH; ++i)
#pragma unroll
      for (int k = 0; k < V; ++k) acc[i][k] *= corr;
#pragma unroll
    for (int u = 0; u < LP_UNROLL; ++u) {
      const float p = expf(sc[u] - m_new);                      // 0 for a key that is not there
      l += p;
#pragma unroll
      for (int i = 0; i < CH; ++i)
#pragma unroll
        for (int k = 0; k < V; ++k) acc[i][k] = fmaf(p, cv[u][i][k], acc[i][k]);
    }
    m = m_new;
  }
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int r = (i * 32 + lane) * V;
    if (r < rank) {
#pragma unroll
      for (int k = 0; k < V; ++k) s_acc[warp * rank + r + k] = acc[i][k];
    }
  }
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < LP_WARPS; ++w) M = fmaxf(M, s_m[w]);
  float f[LP_WARPS], L = 0.f;
#pragma unroll
  for (int w = 0; w < LP_WARPS; ++w) {
    f[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - M);
    L = fmaf(s_l[w], f[w], L);
  }
  float* out = parts + (((size_t)t * H + h) * n_slices + slice) * (rank + 2);
  if (threadIdx.x == 0) { out[0] = M; out[1] = L; }             // an empty slice leaves (-inf, 0, zeros)
  for (int r = threadIdx.x; r < rank; r += blockDim.x) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < LP_WARPS; ++w) a = fmaf(s_acc[w * rank + r], f[w], a);
    out[2 + r] = a;
  }
}

constexpr int LO_COLS = 8;      // value columns of a block of `out` (one warp each)
constexpr int LO_TOKENS = 8;    // tokens whose weighted latents sit in shared memory at a time

template <typename T, int CH>
__global__ void __launch_bounds__(LO_COLS * 32)
latent_out_kernel(const float* __restrict__ parts, const T* __restrict__ w_v, const float* __restrict__ sink,
                  T* __restrict__ out, int ldo, int n_tokens, int H, int dv, int rank, int n_slices) {
  constexpr int V = Vec16<T>::V;
  pdl_launch_dependents();
  extern __shared__ float s_lat[];                              // [LO_TOKENS][rank]
  const int h = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e = blockIdx.y * LO_COLS + warp;
  // this warp's row of Wv_h: a weight, fetched before the wait
  float wv[CH][V];
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int r = (i * 32 + lane) * V;
    if (e < dv && r < rank) {
      Vec16<T>::load(w_v + ((size_t)h * dv + e) * rank + r, wv[i]);
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) wv[i][k] = 0.f;
    }
  }
  const float sk = sink ? sink[h] : -INFINITY;
  pdl_wait();
  for (int t0 = 0; t0 < n_tokens; t0 += LO_TOKENS) {
    const int nt = min(LO_TOKENS, n_tokens - t0);
    __syncthreads();
    for (int tt = warp; tt < nt; tt += LO_COLS) {               // a warp brings a token's slices together
      const float* p = parts + ((size_t)(t0 + tt) * H + h) * n_slices * (rank + 2);
      // lane s holds slice s (at most 32 slices): its maximum and sum, then its factor
      const float ms = lane < n_slices ? p[(size_t)lane * (rank + 2)] : -INFINITY;
      const float ls = lane < n_slices ? p[(size_t)lane * (rank + 2) + 1] : 0.f;
      const float M = fmaxf(warp_max(ms), sk);
      const float es = ms == -INFINITY ? 0.f : expf(ms - M);
      // slices in slice order: lane 0 adds them up one after another
      float L = sink ? expf(sk - M) : 0.f;
      for (int q = 0; q < n_slices; ++q) L = fmaf(__shfl_sync(0xffffffffu, ls, q), __shfl_sync(0xffffffffu, es, q), L);
      const float f = es / L;
#pragma unroll 4      // (several columns' fetches in flight: the loop is a chain of memory latencies otherwise)
      for (int r0 = 0; r0 < rank; r0 += 32) {                  // (the whole warp stays in the loop: it shuffles)
        const int r = r0 + lane;
        const float* col = p + 2 + (r < rank ? r : 0);          // (no branch between the fetches)
        float a = 0.f;
#pragma unroll 4
        for (int q = 0; q < n_slices; ++q)
          a = fmaf(col[(size_t)q * (rank + 2)], __shfl_sync(0xffffffffu, f, q), a);
        if (r < rank) s_lat[tt * rank + r] = a;
      }
    }
    __syncthreads();
    if (e < dv) {
      for (int tt = 0; tt < nt; ++tt) {
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          const int r = (i * 32 + lane) * V;
          if (r < rank) {
#pragma unroll
            for (int k = 0; k < V; ++k) a = fmaf(wv[i][k], s_lat[tt * rank + r + k], a);
          }
        }
        a = warp_sum(a);
        if (lane == 0) out[(size_t)(t0 + tt) * ldo + h * dv + e] = from_float<T>(a);
      }
    }
  }
}

template <typename T, int CH>
static int launch_latent_few(const void* q, int q_is_f32, int ldq, const void* w_k, const void* w_v, const float* sink,
                             const void* pages, const int* page_table, int max_pages, int page_size,
                             const int* seq_slot, const int* token_seq, const int* token_pos, void* out, int ldo,
                             int n_tokens, int H, int dk, int dv, int rank, float scale, int window, int n_slices,
                             float* q_lat, float* parts, cudaStream_t stream) {
  const size_t smem_a = (size_t)(AB_TOKENS * dk + 4 * AB_TOKENS * AB_COLS) * sizeof(float);
  const size_t smem_p = (size_t)LP_WARPS * rank * sizeof(float);
  const size_t smem_o = (size_t)LO_TOKENS * rank * sizeof(float);
  if (smem_a > 48 * 1024 || smem_p > 48 * 1024 || smem_o > 48 * 1024) return DLGO_ERR_SIZE;
  launch_kernel(latent_absorb_kernel<T>, dim3(H, (rank + AB_COLS - 1) / AB_COLS, (n_tokens + AB_TOKENS - 1) / AB_TOKENS), dim3(128),
                smem_a, stream, q, q_is_f32, ldq, (const T*)w_k, q_lat, n_tokens, H, dk, rank);
  int st = launch_status();
  if (st != DLGO_OK) return st;
  launch_kernel(latent_partial_kernel<T, CH>, dim3(n_tokens, H, n_slices), dim3(LP_WARPS * 32), smem_p, stream, q_lat,
                (const T*)pages, page_table, max_pages, page_size, seq_slot, token_seq, token_pos, parts, H, rank,
                n_slices, scale, window);
  st = launch_status();
  if (st != DLGO_OK) return st;
  launch_kernel(latent_out_kernel<T, CH>, dim3(H, (dv + LO_COLS - 1) / LO_COLS), dim3(LO_COLS * 32), smem_o, stream,
                parts, (const T*)w_v, sink, (T*)out, ldo, n_tokens, H, dv, rank, n_slices);
  return launch_status();
}

// ---------------------------------------------------------------------------------------------------------
// Few tokens, every head of a token in one block: the three launches above read every latent row once per head.
// Here a block owns (token, slice of the visible keys) and ALL heads: a tile of 32 latent rows is brought into
// shared memory once (fp32, rows padded so that a lane per key reads 16-byte pieces without bank conflicts) and
// serves every head.  A warp owns HW heads; for the scores a lane owns a key (its dot products with the HW query
// latents, which sit in shared memory and are read as broadcasts), for the weighted latent a lane owns RC columns
// of the row (registers: HW x RC sums).  Online softmax per head in fp32.  Leaves (max, sum, weighted latent) per
// (token, head, slice) in the format of latent_partial.  Then
//   combine  a block per (token, head): the slices meet in slice order (at most 32), the sink joins the
//            denominator; leaves the normalised weighted latent (fp32)
//   project  a block per (head, 16 value columns, 8 tokens): two rows of Wv_h per warp in registers, the weighted
//            latents of several tokens fetched together
constexpr int LT_KEYS = 32, LT_WARPS = 8;

// Row stride of the key tile in floats: a multiple of 4 and odd in 16-byte units, so that a lane per row reads
// 16-byte pieces without bank conflicts.
__host__ __device__ inline int lt_row_stride(int rank) { return rank + ((rank & 7) == 0 ? 4 : 8); }

template <typename T, int RC, int HW>
__global__ void __launch_bounds__(LT_WARPS * 32)
latent_tile_kernel(const float* q_lat, const T* pages, const int* __restrict__ page_table, int max_pages,
                   int page_size, const int* __restrict__ seq_slot, const int* __restrict__ token_seq,
                   const int* __restrict__ token_pos, float* parts, int H, int rank, int n_slices, float scale,
                   int window) {
  constexpr int V = Vec16<T>::V;
  pdl_launch_dependents();
  extern __shared__ __align__(16) float lt_smem[];
  const int RS = lt_row_stride(rank);
  float* q_s = lt_smem;                          // [H][rank]
  float* c_s = q_s + (size_t)H * rank;           // [LT_KEYS][RS]
  float* p_s = c_s + (size_t)LT_KEYS * RS;       // [LT_WARPS * HW][LT_KEYS]
  const int t = blockIdx.x, slice = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = token_pos[t];
  const int* table = page_table + (size_t)seq_slot[token_seq[t]] * max_pages;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int per = (pos - lo + n_slices) / n_slices;             // keys of a slice (the last may have fewer)
  const int j0 = lo + slice * per, j1 = min(pos + 1, j0 + per);
  const int h0 = warp * HW;
  pdl_wait();
  {
    // (four fetches in flight per thread: one after another they would cost a memory latency each)
    const float* qg = q_lat + (size_t)t * H * rank;
    constexpr int STEP = LT_WARPS * 32 * 4;
    for (int i0 = threadIdx.x * 4; i0 < H * rank; i0 += 4 * STEP) {
      float4 tmp[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * STEP < H * rank) tmp[u] = *reinterpret_cast<const float4*>(qg + i0 + u * STEP);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * STEP < H * rank) *reinterpret_cast<float4*>(q_s + i0 + u * STEP) = tmp[u];
    }
  }
  float m[HW], l[HW], acc[HW][RC];
#pragma unroll
  for (int a = 0; a < HW; ++a) {
    m[a] = -INFINITY;
    l[a] = 0.f;
#pragma unroll
    for (int i = 0; i < RC; ++i) acc[a][i] = 0.f;
  }
  const int pieces = rank / V;                  // 16-byte pieces of a row
  for (int jt = j0; jt < j1; jt += LT_KEYS) {
    const int nk = min(LT_KEYS, j1 - jt);
    __syncthreads();                            // (the tile before has been read; q_s is complete)
    for (int idx0 = threadIdx.x; idx0 < LT_KEYS * pieces; idx0 += 4 * LT_WARPS * 32) {
      // four 16-byte pieces in flight per thread; a key beyond the slice's end gives zeros
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = idx0 + u * LT_WARPS * 32;
        const int k = idx / pieces, piece = idx - k * pieces;
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (idx < LT_KEYS * pieces && k < nk) {
          const int j = jt + k;
          const T* row = pages + ((size_t)table[j / page_size] * page_size + j % page_size) * rank;
          raw[u] = *reinterpret_cast<const uint4*>(row + piece * V);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = idx0 + u * LT_WARPS * 32;
        if (idx >= LT_KEYS * pieces) continue;
        const int k = idx / pieces, piece = idx - k * pieces;
        float v[V];
        Vec16<T>::unpack(raw[u], v);
        float* dst = c_s + (size_t)k * RS + piece * V;
#pragma unroll
        for (int e = 0; e < V; e += 4) *reinterpret_cast<float4*>(dst + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
      }
    }
    __syncthreads();
    if (h0 < H) {
      // scores: this lane's key against the warp's heads
      float s[HW];
#pragma unroll
      for (int a = 0; a < HW; ++a) s[a] = 0.f;
      const float4* crow = reinterpret_cast<const float4*>(c_s + (size_t)lane * RS);
      const float4* qrow[HW];
#pragma unroll
      for (int a = 0; a < HW; ++a) qrow[a] = reinterpret_cast<const float4*>(q_s + (size_t)min(h0 + a, H - 1) * rank);
      float s2[HW];                                  // (two chains per head)
#pragma unroll
      for (int a = 0; a < HW; ++a) s2[a] = 0.f;
#pragma unroll 4
      for (int r4 = 0; r4 < (rank >> 2); ++r4) {
        const float4 cv = crow[r4];
#pragma unroll
        for (int a = 0; a < HW; ++a) {
          const float4 qv = qrow[a][r4];
          s[a] = fmaf(qv.x, cv.x, s[a]);
          s2[a] = fmaf(qv.y, cv.y, s2[a]);
          s[a] = fmaf(qv.z, cv.z, s[a]);
          s2[a] = fmaf(qv.w, cv.w, s2[a]);
        }
      }
#pragma unroll
      for (int a = 0; a < HW; ++a) s[a] += s2[a];
      float corr[HW];
#pragma unroll
      for (int a = 0; a < HW; ++a) {
        const float sc = lane < nk ? s[a] * scale : -INFINITY;
        const float m_new = fmaxf(m[a], warp_max(sc));           // finite: the tile holds at least one key
        corr[a] = m[a] == -INFINITY ? 0.f : expf(m[a] - m_new);
        const float pr = lane < nk ? expf(sc - m_new) : 0.f;
        l[a] = fmaf(l[a], corr[a], warp_sum(pr));
        m[a] = m_new;
        p_s[(size_t)(warp * HW + a) * LT_KEYS + lane] = pr;
      }
      __syncwarp();
      // weighted latent: this lane's columns of every row of the tile
#pragma unroll
      for (int a = 0; a < HW; ++a)
#pragma unroll
        for (int i = 0; i < RC; ++i) acc[a][i] *= corr[a];
      const float* ck = c_s + lane;
      const float* pw = p_s + (size_t)warp * HW * LT_KEYS;
#pragma unroll 2
      for (int k = 0; k < nk; ++k, ck += RS) {
        float cv[RC];
#pragma unroll
        for (int i = 0; i < RC; ++i) cv[i] = ck[i * 32];          // (columns beyond the rank read on into the next row,
                                                                  // or behind the tile into p_s: sums that are never stored)
#pragma unroll
        for (int a = 0; a < HW; ++a) {
          const float pk = pw[a * LT_KEYS + k];
#pragma unroll
          for (int i = 0; i < RC; ++i) acc[a][i] = fmaf(pk, cv[i], acc[a][i]);
        }
      }
      __syncwarp();
    }
  }
#pragma unroll
  for (int a = 0; a < HW; ++a) {
    const int h = h0 + a;
    if (h >= H) continue;
    float* out = parts + (((size_t)t * H + h) * n_slices + slice) * (rank + 2);   // an empty slice leaves (-inf, 0, zeros)
    if (lane == 0) { out[0] = m[a]; out[1] = l[a]; }
#pragma unroll
    for (int i = 0; i < RC; ++i) {
      const int r = i * 32 + lane;
      if (r < rank) out[2 + r] = acc[a][i];
    }
  }
}

// lat [T, H, rank]: the slices of (token, head) brought together in slice order and divided by the softmax's sum
__global__ void __launch_bounds__(512)
latent_combine_kernel(const float* parts, const float* __restrict__ sink, float* lat, int H, int rank, int n_slices) {
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y;
  const float* p = parts + ((size_t)t * H + h) * n_slices * (rank + 2);
  const float sk = sink ? sink[h] : -INFINITY;
  __shared__ float f_s[32];                   // a slice's factor: exp(its max - the common max) / the common sum
  pdl_wait();
  if (threadIdx.x < 32) {
    // lane q holds slice q (at most 32 slices); the sum runs in slice order
    const int lane = threadIdx.x;
    const float ms = lane < n_slices ? p[(size_t)lane * (rank + 2)] : -INFINITY;
    const float ls = lane < n_slices ? p[(size_t)lane * (rank + 2) + 1] : 0.f;
    const float M = fmaxf(warp_max(ms), sk);
    const float es = ms == -INFINITY ? 0.f : expf(ms - M);
    float L = sink ? expf(sk - M) : 0.f;
    for (int q = 0; q < n_slices; ++q) L = fmaf(__shfl_sync(0xffffffffu, ls, q), __shfl_sync(0xffffffffu, es, q), L);
    f_s[lane] = es / L;
  }
  __syncthreads();
  float* dst = lat + ((size_t)t * H + h) * rank;
  for (int r = threadIdx.x; r < rank; r += blockDim.x) {
    float a = 0.f;
#pragma unroll 8
    for (int q = 0; q < n_slices; ++q) a = fmaf(p[(size_t)q * (rank + 2) + 2 + r], f_s[q], a);
    dst[r] = a;
  }
}

constexpr int LPJ_COLS = 16;    // value columns of a block of `project` (two per warp)
constexpr int LPJ_TOKENS = 8;   // tokens of a block of `project`

// out[t, h * dv + e] = Wv_h[e, :] . lat[t, h, :]; the rows of TG tokens are fetched together
template <typename T, int RC>
__global__ void __launch_bounds__(256)
latent_project_kernel(const float* lat, const T* __restrict__ w_v, T* out, int ldo, int n_tokens, int H, int dv,
                      int rank) {
  constexpr int TG = RC <= 20 ? 4 : 2;
  pdl_launch_dependents();
  const int h = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e0 = blockIdx.y * LPJ_COLS + warp * 2;
  const int t_begin = blockIdx.z * LPJ_TOKENS, t_end = min(n_tokens, t_begin + LPJ_TOKENS);
  float w0[RC], w1[RC];
#pragma unroll
  for (int i = 0; i < RC; ++i) {
    const int r = i * 32 + lane;
    w0[i] = (e0 < dv && r < rank) ? to_float(w_v[((size_t)h * dv + e0) * rank + r]) : 0.f;
    w1[i] = (e0 + 1 < dv && r < rank) ? to_float(w_v[((size_t)h * dv + e0 + 1) * rank + r]) : 0.f;
  }
  pdl_wait();
  if (e0 >= dv) return;
  for (int tb = t_begin; tb < t_end; tb += TG) {
    float v[TG][RC];
#pragma unroll
    for (int g = 0; g < TG; ++g) {
      const float* row = lat + ((size_t)min(tb + g, t_end - 1) * H + h) * rank;
#pragma unroll
      for (int i = 0; i < RC; ++i) {
        const int r = i * 32 + lane;
        v[g][i] = r < rank ? row[r] : 0.f;
      }
    }
#pragma unroll
    for (int g = 0; g < TG; ++g) {
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int i = 0; i < RC; ++i) {
        a0 = fmaf(w0[i], v[g][i], a0);
        a1 = fmaf(w1[i], v[g][i], a1);
      }
      a0 = warp_sum(a0);
      a1 = warp_sum(a1);
      if (lane == 0 && tb + g < t_end) {
        out[(size_t)(tb + g) * ldo + h * dv + e0] = from_float<T>(a0);
        if (e0 + 1 < dv) out[(size_t)(tb + g) * ldo + h * dv + e0 + 1] = from_float<T>(a1);
      }
    }
  }
}

inline bool latent_tiles_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("DLGO_LATENT_TILES");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

// what the tile kernel keeps in registers: HW heads x RC columns of sums per lane
inline int lt_heads_per_warp(int H) { return H <= 8 ? 1 : (H <= 16 ? 2 : (H <= 32 ? 4 : 0)); }
inline int lt_columns(int rank) { return rank <= 128 ? 4 : (rank <= 256 ? 8 : (rank <= 640 ? 20 : (rank <= 1024 ? 32 : 0))); }
inline size_t lt_smem_bytes(int H, int rank) {
  // (the probabilities' rows come last, 1,024 floats: reads of columns beyond the rank run less than that past the tile)
  return ((size_t)H * rank + (size_t)LT_KEYS * lt_row_stride(rank) + (size_t)LT_WARPS * 4 * LT_KEYS) * sizeof(float);
}
inline bool latent_tiles_takes(int elem_bytes, int H, int rank) {
  const int v = 16 / elem_bytes;
  const int hw = lt_heads_per_warp(H), rc = lt_columns(rank);
  return latent_tiles_enabled() && hw > 0 && rc > 0 && hw * rc <= 80 && rank % v == 0 && rank % 4 == 0 &&
         lt_smem_bytes(H, rank) <= 200 * 1024;
}

template <typename T, int RC, int HW>
static int launch_latent_tile(const float* q_lat, const void* pages, const int* page_table, int max_pages, int page_size,
                              const int* seq_slot, const int* token_seq, const int* token_pos, float* parts,
                              int n_tokens, int H, int rank, int n_slices, float scale, int window,
                              cudaStream_t stream) {
  const size_t smem = lt_smem_bytes(H, rank);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(latent_tile_kernel<T, RC, HW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_kernel(latent_tile_kernel<T, RC, HW>, dim3(n_tokens, n_slices), dim3(LT_WARPS * 32), smem, stream, q_lat,
                (const T*)pages, page_table, max_pages, page_size, seq_slot, token_seq, token_pos, parts, H, rank,
                n_slices, scale, window);
  return launch_status();
}

template <typename T, int RC>
static int launch_latent_tile_by_heads(const float* q_lat, const void* pages, const int* page_table, int max_pages,
                                       int page_size, const int* seq_slot, const int* token_seq, const int* token_pos,
                                       float* parts, int n_tokens, int H, int rank, int n_slices, float scale,
                                       int window, cudaStream_t stream) {
#define LT_ARGS q_lat, pages, page_table, max_pages, page_size, seq_slot, token_seq, token_pos, parts, n_tokens, H, rank, \
                n_slices, scale, window, stream
  const int hw = lt_heads_per_warp(H);
  if (hw == 1) return launch_latent_tile<T, RC, 1>(LT_ARGS);
  if (hw == 2) return launch_latent_tile<T, RC, 2>(LT_ARGS);
  if (hw == 4 && RC <= 20) return launch_latent_tile<T, (RC <= 20 ? RC : 4), 4>(LT_ARGS);
  return DLGO_ERR_SIZE;
#undef LT_ARGS
}

// the four launches: queries into latent space (latent_absorb), tiles, combine, project
template <typename T>
static int launch_latent_tiles(const void* q, int q_is_f32, int ldq, const void* w_k, const void* w_v, const float* sink,
                               const void* pages, const int* page_table, int max_pages, int page_size,
                               const int* seq_slot, const int* token_seq, const int* token_pos, void* out, int ldo,
                               int n_tokens, int H, int dk, int dv, int rank, float scale, int window, int n_slices,
                               float* q_lat, float* parts, cudaStream_t stream) {
  const size_t smem_a = (size_t)(AB_TOKENS * dk + 4 * AB_TOKENS * AB_COLS) * sizeof(float);
  if (smem_a > 48 * 1024) return DLGO_ERR_SIZE;
  launch_kernel(latent_absorb_kernel<T>, dim3(H, (rank + AB_COLS - 1) / AB_COLS, (n_tokens + AB_TOKENS - 1) / AB_TOKENS),
                dim3(128), smem_a, stream, q, q_is_f32, ldq, (const T*)w_k, q_lat, n_tokens, H, dk, rank);
  int st = launch_status();
  if (st != DLGO_OK) return st;
#define LT_ARGS q_lat, pages, page_table, max_pages, page_size, seq_slot, token_seq, token_pos, parts, n_tokens, H, rank, \
                n_slices, scale, window, stream
  const int rc = lt_columns(rank);
  if (rc == 4) st = launch_latent_tile_by_heads<T, 4>(LT_ARGS);
  else if (rc == 8) st = launch_latent_tile_by_heads<T, 8>(LT_ARGS);
  else if (rc == 20) st = launch_latent_tile_by_heads<T, 20>(LT_ARGS);
  else if (rc == 32) st = launch_latent_tile_by_heads<T, 32>(LT_ARGS);
  else return DLGO_ERR_SIZE;
#undef LT_ARGS
  if (st != DLGO_OK) return st;
  // the queries in latent space have been read: their place takes the weighted latents
  launch_kernel(latent_combine_kernel, dim3(n_tokens, H), dim3(rank > 256 ? 512 : (rank > 128 ? 256 : 128)), 0, stream,
                parts, sink, q_lat, H, rank, n_slices);
  st = launch_status();
  if (st != DLGO_OK) return st;
  const dim3 grid(H, (dv + LPJ_COLS - 1) / LPJ_COLS, (n_tokens + LPJ_TOKENS - 1) / LPJ_TOKENS);
  if (rc == 4) launch_kernel(latent_project_kernel<T, 4>, grid, dim3(256), 0, stream, q_lat, (const T*)w_v, (T*)out, ldo, n_tokens, H, dv, rank);
  else if (rc == 8) launch_kernel(latent_project_kernel<T, 8>, grid, dim3(256), 0, stream, q_lat, (const T*)w_v, (T*)out, ldo, n_tokens, H, dv, rank);
  else if (rc == 20) launch_kernel(latent_project_kernel<T, 20>, grid, dim3(256), 0, stream, q_lat, (const T*)w_v, (T*)out, ldo, n_tokens, H, dv, rank);
  else launch_kernel(latent_project_kernel<T, 32>, grid, dim3(256), 0, stream, q_lat, (const T*)w_v, (T*)out, ldo, n_tokens, H, dv, rank);
  return launch_status();
}

template <typename T, int NP>
static int launch_latent(const void* q, int q_is_f32, int ldq, const void* w_k, const void* w_v, const float* sink,
                         const void* pages, const int* page_table, int max_pages, int page_size, const int* seq_slot,
                         const int* token_seq, const int* token_pos, void* out, int ldo, int T_tokens, int H, int dk,
                         int dv, int rank, float scale, int window, cudaStream_t stream) {
  const size_t smem = (size_t)(dk + rank + LA_WARPS * rank) * sizeof(float);
  if (smem > 200 * 1024) return DLGO_ERR_SIZE;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(latent_attention_kernel<T, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_kernel(latent_attention_kernel<T, NP>, dim3(T_tokens, H), dim3(LA_WARPS * 32), smem, stream, q, q_is_f32, ldq,
                (const T*)w_k, (const T*)w_v, sink, (const T*)pages, page_table, max_pages, page_size, seq_slot,
                token_seq, token_pos, (T*)out, ldo, dk, dv, rank, scale, window);
  return launch_status();
}

}  // namespace dlgo

using namespace dlgo;

DLGO_EXPORT int dlgo_latent_norm_append(const float* proj, int ld, int T_tokens, int kv_off, int kv_rank,
                                        const float* w_kv, int q_off, int q_rank, const float* w_q, void* cq,
                                        float eps, const int* token_pos, const int* token_seq, const int* seq_slot,
                                        const int* page_table, int max_pages, void* pages, int dtype, int page_size,
                                        int write_cache, cudaStream_t stream) {
  if (T_tokens <= 0) return DLGO_OK;
  if (kv_rank <= 0 || q_rank < 0 || page_size <= 0) return DLGO_ERR_SIZE;
  const dim3 grid(T_tokens, q_rank > 0 ? 2 : 1);
  const int n = kv_rank > q_rank ? kv_rank : q_rank;
  const int threads = n >= 1024 ? 256 : 128;
  if (dtype == DLGO_F32)
    launch_kernel(latent_norm_append_kernel<float>, grid, dim3(threads), 0, stream, proj, ld, kv_off, kv_rank, w_kv,
                  q_off, q_rank, w_q, (float*)cq, eps, token_pos, token_seq, seq_slot, page_table, max_pages,
                  (float*)pages, page_size, write_cache);
  else if (dtype == DLGO_BF16)
    launch_kernel(latent_norm_append_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, proj, ld, kv_off, kv_rank,
                  w_kv, q_off, q_rank, w_q, (__nv_bfloat16*)cq, eps, token_pos, token_seq, seq_slot, page_table,
                  max_pages, (__nv_bfloat16*)pages, page_size, write_cache);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

DLGO_EXPORT int dlgo_latent_rope_append(float* proj, int ld, int T_tokens, int kv_off, int kv_rank, const float* w_kv,
                                        int q_off, int H, int dq, int rope, const float* freq, float amplitude,
                                        float eps, const int* token_pos, const int* token_seq, const int* seq_slot,
                                        const int* page_table, int max_pages, void* pages, int dtype, int page_size,
                                        int write_cache, cudaStream_t stream) {
  if (T_tokens <= 0) return DLGO_OK;
  if (kv_rank <= 0 || page_size <= 0 || rope <= 0 || (rope & 1) || rope > dq || H <= 0 || freq == nullptr)
    return DLGO_ERR_SIZE;
  const dim3 grid(T_tokens, 2);
  const int threads = kv_rank >= 1024 ? 256 : 128;
  if (dtype == DLGO_F32)
    launch_kernel(latent_rope_append_kernel<float>, grid, dim3(threads), 0, stream, proj, ld, kv_off, kv_rank, w_kv,
                  q_off, H, dq, rope, freq, amplitude, eps, token_pos, token_seq, seq_slot, page_table, max_pages,
                  (float*)pages, page_size, write_cache);
  else if (dtype == DLGO_BF16)
    launch_kernel(latent_rope_append_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, proj, ld, kv_off, kv_rank,
                  w_kv, q_off, H, dq, rope, freq, amplitude, eps, token_pos, token_seq, seq_slot, page_table, max_pages,
                  (__nv_bfloat16*)pages, page_size, write_cache);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

DLGO_EXPORT int dlgo_latent_gather(const void* pages, int dtype, const int* page_table, int max_pages, int page_size,
                                   const int* tmp_pages, int n_tmp, const int* seq_slot, void* out, int rank,
                                   cudaStream_t stream) {
  if (n_tmp <= 0) return DLGO_OK;
  if (rank <= 0 || page_size <= 0) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32)
    launch_kernel(latent_gather_kernel<float>, dim3(n_tmp, GATHER_PARTS), dim3(256), 0, stream, (const float*)pages, page_table,
                  max_pages, page_size, tmp_pages, seq_slot, (float*)out, rank);
  else if (dtype == DLGO_BF16)
    launch_kernel(latent_gather_kernel<__nv_bfloat16>, dim3(n_tmp, GATHER_PARTS), dim3(256), 0, stream, (const __nv_bfloat16*)pages,
                  page_table, max_pages, page_size, tmp_pages, seq_slot, (__nv_bfloat16*)out, rank);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

#define LATENT_ARGS q, q_is_f32, ldq, w_k, w_v, sink, pages, page_table, max_pages, page_size, seq_slot, token_seq, \
                    token_pos, out, ldo, T_tokens, H, dk, dv, rank, scale, window, stream

template <typename T>
static int latent_by_rank(const void* q, int q_is_f32, int ldq, const void* w_k, const void* w_v, const float* sink,
                          const void* pages, const int* page_table, int max_pages, int page_size, const int* seq_slot,
                          const int* token_seq, const int* token_pos, void* out, int ldo, int T_tokens, int H, int dk,
                          int dv, int rank, float scale, int window, cudaStream_t stream) {
  if (rank <= 64) return launch_latent<T, 1>(LATENT_ARGS);
  if (rank <= 128) return launch_latent<T, 2>(LATENT_ARGS);
  if (rank <= 256) return launch_latent<T, 4>(LATENT_ARGS);
  if (rank <= 512) return launch_latent<T, 8>(LATENT_ARGS);
  if (rank <= 1024) return launch_latent<T, 16>(LATENT_ARGS);
  return DLGO_ERR_SIZE;
}

#define FEW_ARGS q, q_is_f32, ldq, w_k, w_v, sink, pages, page_table, max_pages, page_size, seq_slot, token_seq, \
                 token_pos, out, ldo, T_tokens, H, dk, dv, rank, scale, window, n_slices, q_lat, parts, stream

template <typename T>
static int latent_few_by_rank(const void* q, int q_is_f32, int ldq, const void* w_k, const void* w_v,
                              const float* sink, const void* pages, const int* page_table, int max_pages,
                              int page_size, const int* seq_slot, const int* token_seq, const int* token_pos,
                              void* out, int ldo, int T_tokens, int H, int dk, int dv, int rank, float scale,
                              int window, int n_slices, float* q_lat, float* parts, cudaStream_t stream) {
  constexpr int V = 16 / (int)sizeof(T);
  if (rank % V) return DLGO_ERR_SIZE;                           // rows are read 16 bytes at a time
  const int lanes = (rank + V - 1) / V;                         // 16-byte pieces of a row
  if (lanes <= 32) return launch_latent_few<T, 1>(FEW_ARGS);
  if (lanes <= 64) return launch_latent_few<T, 2>(FEW_ARGS);
  if (lanes <= 128) return launch_latent_few<T, 4>(FEW_ARGS);
  if (lanes <= 256) return launch_latent_few<T, 8>(FEW_ARGS);
  return DLGO_ERR_SIZE;
}

// The same attention as three launches (see above) for steps of few tokens: q_lat [T, H, rank] and
// parts [T, H, n_slices, rank + 2] are fp32 scratch; every token's visible keys are cut into n_slices slices.
// 1 if the three-launch kernels take this rank and type (rows read 16 bytes at a time)
DLGO_EXPORT int dlgo_latent_attention_few_takes(int dtype, int rank) {
  const int v = dtype == DLGO_F32 ? 4 : 8;
  return (dtype == DLGO_F32 || dtype == DLGO_BF16) && rank % v == 0 && rank <= 256 * v;
}

DLGO_EXPORT int dlgo_latent_attention_few(const void* q, int q_is_f32, int ldq, const void* w_k, const void* w_v,
                                          const float* sink, const void* pages, int dtype, const int* page_table,
                                          int max_pages, int page_size, const int* seq_slot, const int* token_seq,
                                          const int* token_pos, void* out, int ldo, int T_tokens, int H, int dk,
                                          int dv, int rank, float scale, int window, int n_slices, float* q_lat,
                                          float* parts, cudaStream_t stream) {
  if (T_tokens <= 0) return DLGO_OK;
  if (H <= 0 || dk <= 0 || dv <= 0 || rank <= 0 || page_size <= 0 || window < 0 || n_slices < 1 ||
      n_slices > 32 || H > 65535)      // (a lane per slice where the slices meet)
    return DLGO_ERR_SIZE;
  if (((uintptr_t)pages & 15) || ((uintptr_t)w_v & 15)) return DLGO_ERR_ALIGN;
  if (dtype == DLGO_F32) return latent_few_by_rank<float>(FEW_ARGS);
  if (dtype == DLGO_BF16) {
    return latent_few_by_rank<__nv_bfloat16>(FEW_ARGS);
  }
  return DLGO_ERR_DTYPE;
}

// The same through tiles of keys that serve all heads (four launches); `takes` says whether the sizes fit.
DLGO_EXPORT int dlgo_latent_attention_tiles_takes(int dtype, int H, int rank) {
  if (dtype != DLGO_F32 && dtype != DLGO_BF16) return 0;
  return latent_tiles_takes(dtype == DLGO_F32 ? 4 : 2, H, rank) ? 1 : 0;
}

DLGO_EXPORT int dlgo_latent_attention_tiles(const void* q, int q_is_f32, int ldq, const void* w_k, const void* w_v,
                                            const float* sink, const void* pages, int dtype, const int* page_table,
                                            int max_pages, int page_size, const int* seq_slot, const int* token_seq,
                                            const int* token_pos, void* out, int ldo, int T_tokens, int H, int dk,
                                            int dv, int rank, float scale, int window, int n_slices, float* q_lat,
                                            float* parts, cudaStream_t stream) {
  if (T_tokens <= 0) return DLGO_OK;
  if (H <= 0 || dk <= 0 || dv <= 0 || rank <= 0 || page_size <= 0 || window < 0 || n_slices < 1 || n_slices > 32 ||
      H > 65535 || !dlgo_latent_attention_tiles_takes(dtype, H, rank))
    return DLGO_ERR_SIZE;
  if (((uintptr_t)pages & 15) || ((uintptr_t)q_lat & 15)) return DLGO_ERR_ALIGN;
#define TILES_ARGS q, q_is_f32, ldq, w_k, w_v, sink, pages, page_table, max_pages, page_size, seq_slot, token_seq, \
                   token_pos, out, ldo, T_tokens, H, dk, dv, rank, scale, window, n_slices, q_lat, parts, stream
  if (dtype == DLGO_F32) return launch_latent_tiles<float>(TILES_ARGS);
  return launch_latent_tiles<__nv_bfloat16>(TILES_ARGS);
#undef TILES_ARGS
}

// q [T, >= H*dk] (fp32 or the cache's type), w_k [H*dk, rank], w_v [H*dv, rank], pages [n, page_size, rank],
// out [T, >= H*dv]; sink [H] fp32 or null; window 0: every earlier key
DLGO_EXPORT int dlgo_latent_attention(const void* q, int q_is_f32, int ldq, const void* w_k, const void* w_v,
                                      const float* sink, const void* pages, int dtype, const int* page_table,
                                      int max_pages, int page_size, const int* seq_slot, const int* token_seq,
                                      const int* token_pos, void* out, int ldo, int T_tokens, int H, int dk, int dv,
                                      int rank, float scale, int window, cudaStream_t stream) {
  if (T_tokens <= 0) return DLGO_OK;
  if (H <= 0 || dk <= 0 || dv <= 0 || rank <= 0 || page_size <= 0 || window < 0) return DLGO_ERR_SIZE;
  if (((uintptr_t)pages & 7) || ((uintptr_t)w_v & 7)) return DLGO_ERR_ALIGN;
  if (dtype == DLGO_F32) return latent_by_rank<float>(LATENT_ARGS);
  if (dtype == DLGO_BF16) {
    return latent_by_rank<__nv_bfloat16>(LATENT_ARGS);
  }
  return DLGO_ERR_DTYPE;
}
