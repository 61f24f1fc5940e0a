// Time mixing: a per-head recurrence over a fixed-size state whose decay depends on the token, per key channel,
// with a bonus for the current token, fed by projections that each read their own blend of this token's input and
// the previous token's.
//
//   blend s:   m_s[t] = h[t] + (h[t-1] - h[t]) * mu_s           h[-1] = 0 at a sequence's start; between steps the
//                                                               last input of a sequence is kept in its state row
//   decay:     w_t = exp(-exp(z_t + w0))                        z_t the result of the decay's own small projection
//   per head:  o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t        S [n, n] fp32, zero at a sequence's start
//              S_t = diag(w_t) S_(t-1) + k_t v_t^T
//
// A sequence's state row is [H * n * n numbers of S | d numbers of the last input], fp32, `state_ld` floats apart.
//
// token_shift_mix: the blends, from the fp32 residual stream, into the run's type, one [T, d] matrix per blend.
// wkv_scan:        any head size: a block per (sequence, head, run of value columns), its part of S in shared memory.
// wkv_segments:    head sizes 32 / 64 / 128: a thread keeps its column of S in registers, and a sequence's tokens of
//                  one step are cut into segments that run side by side:
//                    pass 1: every segment runs from a zero state and leaves its end state L_j and the product P_j of
//                            its tokens' decays (per key channel); a sequence's first segment copies the stored state
//                    pass 2: segment j starts from S_in carried through the segments before it
//                            (S <- diag(P_m) S + L_m for m before j), walks its tokens and writes their outputs
//                  With one segment per sequence (decoding, short prompts) pass 2 runs alone from the stored state.
// Decays, exponentials, state and outputs are fp32 in every precision.
#include "common.cuh"
#include "async_copy.cuh"

namespace dlgo {

template <typename TO>
__global__ void token_shift_mix_kernel(const float* x, const float* __restrict__ mu, int n_mix,
                                       const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                       const float* state, long long state_ld, int prev_off,
                                       TO* out, int T, int d) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int seq = token_seq[t];
  const bool first = t == 0 || token_seq[t - 1] != seq;       // the sequence's first token of this step
  const int slot = seq_slot[seq];
  pdl_wait();
  const float* cur = x + (size_t)t * d;
  const float* prev = first ? state + (size_t)slot * state_ld + prev_off : x + (size_t)(t - 1) * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float a = cur[i], dlt = prev[i] - a;
    for (int s = 0; s < n_mix; ++s)
      out[((size_t)s * T + t) * d + i] = from_float<TO>(fmaf(dlt, mu[(size_t)s * d + i], a));
  }
}

__device__ __forceinline__ float decay_of(float z, float w0) { return expf(-expf(z + w0)); }

// the last input of a sequence's tokens of this step into its state row (the part of d that block `part` of `parts` owns)
__device__ __forceinline__ void keep_last_input(const float* x, int d, int last_tok, float* st_prev, int part,
                                                int parts) {
  if (x == nullptr) return;
  for (int i = part * blockDim.x + threadIdx.x; i < d; i += parts * blockDim.x) st_prev[i] = x[(size_t)last_tok * d + i];
}

__global__ void wkv_scan_kernel(const float* r, const float* k, const float* v, const float* zw, int ld,
                                const float* __restrict__ w0,
                                const float* __restrict__ u, const int* __restrict__ tiles,
                                const int* __restrict__ seq_slot, float* state, long long state_ld, const float* x,
                                int d, float* out, int H, int n, int dvc) {
  pdl_launch_dependents();
  extern __shared__ float smem[];
  const int e0 = blockIdx.z * dvc, nc = min(dvc, n - e0);
  float* S = smem;                          // [n][nc]
  float* us = S + (size_t)n * dvc;          // [n]
  float* buf = us + n;                      // two buffers of [r (n) | k (n) | w (n) | v (nc)]
  const int per = 3 * n + dvc;
  const int h = blockIdx.y;
  const int seq = tiles[blockIdx.x * 3 + 0], first = tiles[blockIdx.x * 3 + 1], count = tiles[blockIdx.x * 3 + 2];
  const int slot = seq_slot[seq];
  float* st = state + (size_t)slot * state_ld + (size_t)h * n * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) us[i] = u[h * n + i];
  pdl_wait();
  for (int i = threadIdx.x; i < n * nc; i += blockDim.x) S[i] = st[(size_t)(i / nc) * n + e0 + i % nc];
  auto fetch = [&](int tok, float* b) {
    const size_t row = (size_t)tok * ld + (size_t)h * n;
    for (int i = threadIdx.x; i < 3 * n + nc; i += blockDim.x) {
      float val;
      if (i < n) val = r[row + i];
      else if (i < 2 * n) val = k[row + i - n];
      else if (i < 3 * n) val = decay_of(zw[row + i - 2 * n], w0[h * n + i - 2 * n]);
      else val = v[row + e0 + (i - 3 * n)];
      b[i] = val;
    }
  };
  fetch(first, buf);
  __syncthreads();
  for (int t = 0; t < count; ++t) {
    float* cur = buf + (t & 1) * per;
    if (t + 1 < count) fetch(first + t + 1, buf + ((t + 1) & 1) * per);
    const float* sr = cur;
    const float* sk = cur + n;
    const float* sw = cur + 2 * n;
    const float* sv = cur + 3 * n;
    for (int e = threadIdx.x; e < nc; e += blockDim.x) {
      const float val = sv[e];
      float o = 0.f;
      for (int i = 0; i < n; ++i) {
        const float s = S[i * nc + e], kv = sk[i] * val;
        o = fmaf(sr[i], fmaf(us[i], kv, s), o);
        S[i * nc + e] = fmaf(sw[i], s, kv);
      }
      out[(size_t)(first + t) * ld + h * n + e0 + e] = o;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < n * nc; i += blockDim.x) st[(size_t)(i / nc) * n + e0 + i % nc] = S[i];
  if (blockIdx.z == 0) keep_last_input(x, d, first + count - 1, state + (size_t)slot * state_ld + (size_t)H * n * n, h, H);
}

enum { WKV_DIRECT = 0, WKV_LOCAL = 1, WKV_CARRY = 2 };

constexpr int WKV_CHUNK = 8;     // tokens that are fetched together, one chunk ahead of the products

// A block of DK threads per (segment, head): thread e keeps column e of the state in registers and owns decay
// channel e.  A token's r | k | z | v (4 DK numbers) come in chunks of WKV_CHUNK tokens through a ring of two
// shared-memory buffers filled by asynchronous copies, so that a token's products never wait for memory; when a
// chunk has landed its z become decays in place (thread e: channel e of every token).
template <int DK, int MODE>
__global__ void __launch_bounds__(DK)
wkv_segments_kernel(const float* r, const float* k, const float* v, const float* zw, int ld,
                    const float* __restrict__ w0, const float* __restrict__ u,
                    const int* __restrict__ tiles, int n_tiles, const int* __restrict__ seq_slot,
                    float* state, long long state_ld, const float* x, int d, float* local, float* start_copy,
                    float* decays, float* out, int H) {
  pdl_launch_dependents();
  constexpr int dv = DK, CH = WKV_CHUNK, ROW = 4 * DK, PIECES = DK / 4;
  __shared__ __align__(16) float ring[2][CH * ROW];
  __shared__ __align__(16) float us[DK];
  const int tile = blockIdx.x, h = blockIdx.y;
  const int e = threadIdx.x;                                     // this thread's column of the state, and its channel
  const int seq = tiles[tile * 3 + 0], first = tiles[tile * 3 + 1], count = tiles[tile * 3 + 2];
  const int slot = seq_slot[seq];
  int t0 = tile;                                                 // the sequence's first segment
  while (t0 > 0 && tiles[(t0 - 1) * 3] == seq) --t0;
  const bool last = tile + 1 == n_tiles || tiles[(tile + 1) * 3] != seq;
  float* st = state + (size_t)slot * state_ld + (size_t)h * DK * dv;
  const size_t seg_elems = (size_t)H * DK * dv;
  us[e] = u[h * DK + e];
  const float w0_mine = w0[h * DK + e];
  pdl_wait();
  auto load_chunk = [&](int c, float* buf) {
    const int tok0 = first + c * CH, nt = min(CH, count - c * CH);
    for (int i = threadIdx.x; i < nt * 4 * PIECES; i += DK) {
      const int t = i / (4 * PIECES), a = (i / PIECES) & 3, p = i % PIECES;
      const float* src = a == 0 ? r : (a == 1 ? k : (a == 2 ? zw : v));
      copy16_async(buf + t * ROW + a * DK + p * 4, src + (size_t)(tok0 + t) * ld + (size_t)h * DK + p * 4);
    }
    copies_commit();
  };
  const int n_chunks = (count + CH - 1) / CH;
  load_chunk(0, ring[0]);
  float S[DK];
  if (MODE == WKV_LOCAL) {
    if (tile == t0) {                                            // (all loads first: the copy's stores do not wait for them one by one)
#pragma unroll
      for (int i = 0; i < DK; ++i) S[i] = st[(size_t)i * dv + e];
#pragma unroll
      for (int i = 0; i < DK; ++i) start_copy[(size_t)tile * seg_elems + ((size_t)h * DK + i) * dv + e] = S[i];
    }
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = 0.f;
  } else if (MODE == WKV_DIRECT) {
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = st[(size_t)i * dv + e];
  } else {
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = start_copy[(size_t)t0 * seg_elems + ((size_t)h * DK + i) * dv + e];
    for (int j = t0; j < tile; ++j) {
      const float* L = local + (size_t)j * seg_elems + (size_t)h * DK * dv;
      const float* P = decays + ((size_t)j * H + h) * DK;
#pragma unroll
      for (int i = 0; i < DK; ++i) S[i] = fmaf(P[i], S[i], L[(size_t)i * dv + e]);
    }
  }
  float prod = 1.0f;                                             // product of this segment's decays in channel e
  for (int c = 0; c < n_chunks; ++c) {
    float* buf = ring[c & 1];
    if (c + 1 < n_chunks) {
      load_chunk(c + 1, ring[(c + 1) & 1]);                      // (its last readers passed the barrier that ended chunk c - 1)
      copies_wait<1>();
    } else {
      copies_wait<0>();
    }
    __syncthreads();
    const int nt = min(CH, count - c * CH);
    for (int t = 0; t < nt; ++t) {
      const float w = decay_of(buf[t * ROW + 2 * DK + e], w0_mine);
      buf[t * ROW + 2 * DK + e] = w;
      if (MODE == WKV_LOCAL) prod *= w;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float* cur = buf + t * ROW;
      const float val = cur[3 * DK + e];
      float o0 = 0.f, o1 = 0.f;                                   // two chains of sums; more of them cost registers that a 128-wide state needs
#pragma unroll
      for (int i = 0; i < DK; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(cur + DK + i);
        const float4 w4 = *reinterpret_cast<const float4*>(cur + 2 * DK + i);
        const float kv0 = k4.x * val, kv1 = k4.y * val, kv2 = k4.z * val, kv3 = k4.w * val;
        if (MODE != WKV_LOCAL) {
          const float4 r4 = *reinterpret_cast<const float4*>(cur + i);
          const float4 u4 = *reinterpret_cast<const float4*>(us + i);
          o0 = fmaf(r4.x, fmaf(u4.x, kv0, S[i]), o0);
          o1 = fmaf(r4.y, fmaf(u4.y, kv1, S[i + 1]), o1);
          o0 = fmaf(r4.z, fmaf(u4.z, kv2, S[i + 2]), o0);
          o1 = fmaf(r4.w, fmaf(u4.w, kv3, S[i + 3]), o1);
        }
        S[i] = fmaf(w4.x, S[i], kv0);
        S[i + 1] = fmaf(w4.y, S[i + 1], kv1);
        S[i + 2] = fmaf(w4.z, S[i + 2], kv2);
        S[i + 3] = fmaf(w4.w, S[i + 3], kv3);
      }
      if (MODE != WKV_LOCAL) out[(size_t)(first + c * CH + t) * ld + h * DK + e] = o0 + o1;
    }
    __syncthreads();                                             // the buffer is free for the chunk after next
  }
  if (MODE == WKV_LOCAL) {
    decays[((size_t)tile * H + h) * DK + e] = prod;
    float* L = local + (size_t)tile * seg_elems + (size_t)h * DK * dv;
#pragma unroll
    for (int i = 0; i < DK; ++i) L[(size_t)i * dv + e] = S[i];
    return;
  }
  if (last) {
#pragma unroll
    for (int i = 0; i < DK; ++i) st[(size_t)i * dv + e] = S[i];
    keep_last_input(x, d, first + count - 1, state + (size_t)slot * state_ld + (size_t)H * DK * dv, h, H);
  }
}

template <int DK>
static int launch_wkv_segments(const float* r, const float* k, const float* v, const float* zw, int ld, const float* w0,
                               const float* u, const int* tiles, int n_tiles, int direct, const int* seq_slot,
                               float* state, long long state_ld, const float* x, int d, float* scratch, float* out,
                               int H, cudaStream_t stream) {
  const dim3 grid(n_tiles, H), block(DK);
  const size_t seg = (size_t)n_tiles * H * DK * DK;
  float* local = scratch;
  float* start_copy = scratch ? scratch + seg : nullptr;
  float* decays = scratch ? scratch + 2 * seg : nullptr;
  if (direct) {
    launch_kernel(wkv_segments_kernel<DK, WKV_DIRECT>, grid, block, 0, stream, r, k, v, zw, ld, w0, u, tiles, n_tiles,
                  seq_slot, state, state_ld, x, d, local, start_copy, decays, out, H);
    return launch_status();
  }
  if (!scratch) return DLGO_ERR_SIZE;
  launch_kernel(wkv_segments_kernel<DK, WKV_LOCAL>, grid, block, 0, stream, r, k, v, zw, ld, w0, u, tiles, n_tiles,
                seq_slot, state, state_ld, x, d, local, start_copy, decays, out, H);
  int st = launch_status();
  if (st != DLGO_OK) return st;
  launch_kernel(wkv_segments_kernel<DK, WKV_CARRY>, grid, block, 0, stream, r, k, v, zw, ld, w0, u, tiles, n_tiles,
                seq_slot, state, state_ld, x, d, local, start_copy, decays, out, H);
  return launch_status();
}

}  // namespace dlgo

using namespace dlgo;

// x [T, d] fp32; mu [n_mix, d] fp32; state rows `state_ld` floats apart with the last input at `prev_off`;
// out [n_mix, T, d] in `dtype`
DLGO_EXPORT int dlgo_token_shift_mix(const float* x, const float* mu, int n_mix, const int* token_seq,
                                     const int* seq_slot, const float* state, long long state_ld, int prev_off, void* out,
                                     int dtype, int T, int d, cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (d <= 0 || n_mix <= 0) return DLGO_ERR_SIZE;
  const int threads = d >= 1024 ? 256 : 128;
  if (dtype == DLGO_F32)
    launch_kernel(token_shift_mix_kernel<float>, dim3(T), dim3(threads), 0, stream, x, mu, n_mix, token_seq, seq_slot,
                  state, state_ld, prev_off, (float*)out, T, d);
  else if (dtype == DLGO_BF16)
    launch_kernel(token_shift_mix_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, x, mu, n_mix, token_seq,
                  seq_slot, state, state_ld, prev_off, (__nv_bfloat16*)out, T, d);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

DLGO_EXPORT int dlgo_wkv_segments_takes(int n) { return n == 32 || n == 64 || n == 128; }

// r, k, v, zw [T, ld] fp32 (heads side by side, n numbers each; ld = H * n); w0 [H * n], u [H * n] fp32;
// tiles [n_tiles, 3] (sequence, first packed token, count), a sequence's segments side by side in token order;
// state rows [H * n * n | d]; x [T, d] fp32 (the inputs whose last row per sequence is kept; may be null);
// out [T, ld] fp32.  `direct`: one segment per sequence; else scratch holds n_tiles * H * (2 n n + n) floats.
DLGO_EXPORT int dlgo_wkv_segments(const float* r, const float* k, const float* v, const float* zw, int ld,
                                  const float* w0, const float* u, const int* tiles, int n_tiles, int direct,
                                  const int* seq_slot, float* state, long long state_ld, const float* x, int d,
                                  float* scratch, float* out, int H, int n, cudaStream_t stream) {
  if (n_tiles <= 0) return DLGO_OK;
  if (H <= 0 || H > 65535) return DLGO_ERR_SIZE;
  // rows are fetched in 16-byte pieces
  if ((((size_t)r | (size_t)k | (size_t)v | (size_t)zw) & 15) || (ld & 3)) return DLGO_ERR_SIZE;
#define WKV_ARGS r, k, v, zw, ld, w0, u, tiles, n_tiles, direct, seq_slot, state, state_ld, x, d, scratch, out, H, stream
  if (n == 32) return launch_wkv_segments<32>(WKV_ARGS);
  if (n == 64) return launch_wkv_segments<64>(WKV_ARGS);
  if (n == 128) return launch_wkv_segments<128>(WKV_ARGS);
  return DLGO_ERR_SIZE;
}

// The same for any head size, one row of `tiles` per sequence of the step.
DLGO_EXPORT int dlgo_wkv_scan(const float* r, const float* k, const float* v, const float* zw, int ld, const float* w0,
                              const float* u, const int* tiles, int n_seqs, const int* seq_slot, float* state,
                              long long state_ld, const float* x, int d, float* out, int H, int n, cudaStream_t stream) {
  if (n_seqs <= 0) return DLGO_OK;
  if (H <= 0 || H > 65535 || n <= 0) return DLGO_ERR_SIZE;
  int dvc = n;
  auto bytes = [&](int c) { return ((size_t)n * c + n + 2 * (3 * (size_t)n + c)) * sizeof(float); };
  while (dvc > 1 && bytes(dvc) > 96 * 1024) dvc = (dvc + 1) / 2;
  const size_t smem = bytes(dvc);
  if (smem > 200 * 1024) return DLGO_ERR_SIZE;
  if (smem > 48 * 1024) cudaFuncSetAttribute(wkv_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int threads = ((dvc + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  if (threads < 64) threads = 64;
  launch_kernel(wkv_scan_kernel, dim3(n_seqs, H, (n + dvc - 1) / dvc), dim3(threads), smem, stream, r, k, v, zw, ld, w0, u,
                tiles, seq_slot, state, state_ld, x, d, out, H, n, dvc);
  return launch_status();
}
