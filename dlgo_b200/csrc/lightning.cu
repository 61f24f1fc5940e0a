// Linear attention with a per-head decay ("lightning attention"), as a recurrence over a fixed-size state.
//
// Per head, with q_t = a(Wq h_t), k_t = a(Wk h_t) (dk numbers) and v_t = a(Wv h_t) (dv numbers), where a is silu
// (`act` 1) or nothing (`act` 0: the caller has prepared q and k, e.g. rotated and scaled them):
//   S_t = lambda * S_(t-1) + k_t v_t^T          S is [dk, dv], fp32, zero at a sequence's start
//   o_t = S_t^T q_t
// The state of a sequence lives in its slot of the state area between steps, so a prompt may arrive in any
// number of portions and decoding continues where the prompt stopped.
//
// lightning_scan: one block per (sequence, head, run of value columns); its part of the state sits in shared
// memory while the block walks the sequence's tokens of this step in order.  The projections arrive as fp32 rows [q | k | v | ...]; activation,
// decay, state and output are fp32.
#include "common.cuh"
#include "async_copy.cuh"

namespace dlgo {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

__global__ void lightning_scan_kernel(const float* proj, int ld, int q_off, int k_off, int v_off,
                                      const int* __restrict__ tiles, const int* __restrict__ seq_slot,
                                      const float* __restrict__ decay, float* state,
                                      float* out, int ldo, int H, int dk, int dv, int dvc, int act) {
  pdl_launch_dependents();
  extern __shared__ float smem[];
  // the block's columns [e0, e0 + n) of the state (columns are independent of one another)
  const int e0 = blockIdx.z * dvc, n = min(dvc, dv - e0);
  float* S = smem;                       // [dk][n]
  float* qk = S + (size_t)dk * dvc;      // two buffers of [q (dk) | k (dk) | v (n)]
  const int per = 2 * dk + dvc;
  const int h = blockIdx.y;
  const int seq = tiles[blockIdx.x * 3 + 0], first = tiles[blockIdx.x * 3 + 1], count = tiles[blockIdx.x * 3 + 2];
  const int slot = seq_slot[seq];
  const float lam = decay[h];
  float* st = state + ((size_t)slot * H + h) * dk * dv;
  pdl_wait();
  for (int i = threadIdx.x; i < dk * n; i += blockDim.x) S[i] = st[(size_t)(i / n) * dv + e0 + i % n];
  auto fetch = [&](int tok, float* buf) {
    const float* row = proj + (size_t)tok * ld;
    for (int i = threadIdx.x; i < 2 * dk + n; i += blockDim.x) {
      const int col = i < dk ? q_off + h * dk + i : (i < 2 * dk ? k_off + h * dk + (i - dk) : v_off + h * dv + e0 + (i - 2 * dk));
      buf[i] = act ? silu_f(row[col]) : row[col];
    }
  };
  fetch(first, qk);
  __syncthreads();
  for (int t = 0; t < count; ++t) {
    float* cur = qk + (t & 1) * per;
    if (t + 1 < count) fetch(first + t + 1, qk + ((t + 1) & 1) * per);
    const float* sq = cur;
    const float* sk = cur + dk;
    const float* sv = cur + 2 * dk;
    // a thread owns columns e of the state: no two threads touch the same element
    for (int e = threadIdx.x; e < n; e += blockDim.x) {
      const float v = sv[e];
      float o = 0.f;
      for (int i = 0; i < dk; ++i) {
        const float s = fmaf(lam, S[i * n + e], sk[i] * v);
        S[i * n + e] = s;
        o = fmaf(s, sq[i], o);
      }
      out[(size_t)(first + t) * ldo + h * dv + e0 + e] = o;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < dk * n; i += blockDim.x) st[(size_t)(i / n) * dv + e0 + i % n] = S[i];
}

// Queries and keys made ready for the recurrence, in place in the fp32 projection rows: among the first `rot`
// numbers of every head, number i turns with number i + rot/2 by the angle float(position) * freq[i] (formed, like
// its cosine and sine, in fp32); keys are then multiplied by `k_scale`.  A warp per (token, q or k head).
constexpr int RS_WARPS = 4;
__global__ void __launch_bounds__(RS_WARPS * 32)
rotate_scale_kernel(float* proj, int ld, int q_off, int k_off, const float* __restrict__ freq, int rot,
                    const int* __restrict__ token_pos, int T, int H, int dk, float k_scale) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long item = (long long)blockIdx.x * RS_WARPS + warp;
  if (item >= (long long)T * 2 * H) return;
  const int t = (int)(item / (2 * H)), hh = (int)(item - (long long)t * 2 * H);
  const bool is_k = hh >= H;
  const int h = is_k ? hh - H : hh;
  const float p = (float)token_pos[t];
  const float sc = is_k ? k_scale : 1.0f;
  pdl_wait();
  float* u = proj + (size_t)t * ld + (is_k ? k_off : q_off) + (size_t)h * dk;
  const int rh = rot / 2;
  for (int i = lane; i < rh; i += 32) {
    const float a = u[i], b = u[i + rh];
    float sn, cs;
    sincosf(p * freq[i], &sn, &cs);
    u[i] = (a * cs - b * sn) * sc;
    u[i + rh] = (b * cs + a * sn) * sc;
  }
  if (is_k && sc != 1.0f)
    for (int i = rot + lane; i < dk; i += 32) u[i] *= sc;
}

// Common qk sizes: a thread keeps its column of the state in registers, and a sequence's tokens of one step
// are cut into segments that run side by side.
//   pass 1 (LOCAL): every segment runs from a zero state and leaves its end state L_i; a sequence's first
//                   segment also copies the sequence's stored state S_in aside
//   pass 2:         segment i starts from  lambda^(n_0 + .. + n_(i-1)) S_in + sum_(j<i) lambda^(n_(j+1) + .. + n_(i-1)) L_j,
//                   walks its tokens and writes their outputs; the last segment stores the sequence's new state
// With DIRECT (one segment per sequence: decoding, short prompts) pass 2 runs alone and starts from S_in.
// A token's q | k (2 DK numbers) and the block's up to 128 value columns come in chunks of SEG_CHUNK tokens through
// a ring of two shared-memory buffers filled by asynchronous copies, one chunk ahead of the products, so that a
// token's products never wait for memory (`vec`: every piece starts on a 16-byte boundary; else 4-byte copies).
constexpr int SEG_CHUNK = 8;

template <int DK, bool LOCAL, bool DIRECT>
__global__ void __launch_bounds__(128)
lightning_segments_kernel(const float* proj, int ld, int q_off, int k_off, int v_off,
                          const int* __restrict__ tiles, int n_tiles, const int* __restrict__ seq_slot,
                          const float* __restrict__ decay, float* state, float* local,
                          float* start_copy, float* out, int ldo, int H, int dv, int act, int vec) {
  pdl_launch_dependents();
  constexpr int CH = SEG_CHUNK, ROW = 2 * DK + 128;
  __shared__ __align__(16) float ring[2][CH * ROW];
  const int tile = blockIdx.x, h = blockIdx.y;
  const int e0 = blockIdx.z * 128;                               // the block's first column of the state
  const int e = e0 + threadIdx.x;                                // this thread's column
  const int nv = min(128, dv - e0);
  const bool live = e < dv;
  const int seq = tiles[tile * 3 + 0], first = tiles[tile * 3 + 1], count = tiles[tile * 3 + 2];
  const int slot = seq_slot[seq];
  const float lam = decay[h];
  int t0 = tile;                                                 // the sequence's first segment
  while (t0 > 0 && tiles[(t0 - 1) * 3] == seq) --t0;
  const bool last = tile + 1 == n_tiles || tiles[(tile + 1) * 3] != seq;
  float* st = state + ((size_t)slot * H + h) * DK * dv;
  const size_t seg_elems = (size_t)H * DK * dv;
  pdl_wait();
  auto load_chunk = [&](int c, float* buf) {
    const int tok0 = first + c * CH, nt = min(CH, count - c * CH);
    // a row of the buffer: q, k, then the block's value columns; piece p of a row lands at the same place p
    const int unit = vec ? 4 : 1, per = (2 * DK + nv) / unit, nq = DK / unit;
    for (int i = threadIdx.x; i < nt * per; i += 128) {
      const int t = i / per, p = i - t * per;
      const float* row = proj + (size_t)(tok0 + t) * ld;
      const float* src = p < nq ? row + q_off + h * DK + p * unit
                       : p < 2 * nq ? row + k_off + h * DK + (p - nq) * unit
                                    : row + v_off + h * dv + e0 + (p - 2 * nq) * unit;
      if (vec) copy16_async(buf + t * ROW + p * 4, src);
      else copy4_async(buf + t * ROW + p, src);
    }
    copies_commit();
  };
  const int n_chunks = (count + CH - 1) / CH;
  load_chunk(0, ring[0]);
  float S[DK];
  if (LOCAL) {
    if (tile == t0 && live) {                                    // (all loads first: the copy's stores do not wait for them one by one)
#pragma unroll
      for (int i = 0; i < DK; ++i) S[i] = st[(size_t)i * dv + e];
#pragma unroll
      for (int i = 0; i < DK; ++i) start_copy[(size_t)tile * seg_elems + ((size_t)h * DK + i) * dv + e] = S[i];
    }
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = 0.f;
  } else if (DIRECT) {
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = live ? st[(size_t)i * dv + e] : 0.f;
  } else {
    int before = 0;                                              // tokens of this step ahead of the segment
    for (int j = t0; j < tile; ++j) before += tiles[j * 3 + 2];
    const float f0 = powf(lam, (float)before);
#pragma unroll
    for (int i = 0; i < DK; ++i)
      S[i] = live ? f0 * start_copy[(size_t)t0 * seg_elems + ((size_t)h * DK + i) * dv + e] : 0.f;
    int after = before;
    for (int j = t0; j < tile; ++j) {
      after -= tiles[j * 3 + 2];                                 // tokens between segment j's end and this one's start
      const float f = powf(lam, (float)after);
      const float* L = local + (size_t)j * seg_elems + (size_t)h * DK * dv;
      if (live) {
#pragma unroll
        for (int i = 0; i < DK; ++i) S[i] = fmaf(f, L[(size_t)i * dv + e], S[i]);
      }
    }
  }
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
    if (act) {                                                   // silu on q, k and v where they landed
      for (int i = threadIdx.x; i < nt * ROW; i += 128) {
        const int p = i % ROW;
        if (p < 2 * DK + nv) buf[i] = silu_f(buf[i]);
      }
      __syncthreads();
    }
    for (int t = 0; t < nt; ++t) {
      const float* cur = buf + t * ROW;
      const float v = live ? cur[2 * DK + threadIdx.x] : 0.f;
      float o0 = 0.f, o1 = 0.f;                                  // two chains of sums
#pragma unroll
      for (int i = 0; i < DK; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(cur + DK + i);
        S[i] = fmaf(lam, S[i], k4.x * v);
        S[i + 1] = fmaf(lam, S[i + 1], k4.y * v);
        S[i + 2] = fmaf(lam, S[i + 2], k4.z * v);
        S[i + 3] = fmaf(lam, S[i + 3], k4.w * v);
        if (!LOCAL) {
          const float4 q4 = *reinterpret_cast<const float4*>(cur + i);
          o0 = fmaf(S[i], q4.x, o0);
          o1 = fmaf(S[i + 1], q4.y, o1);
          o0 = fmaf(S[i + 2], q4.z, o0);
          o1 = fmaf(S[i + 3], q4.w, o1);
        }
      }
      if (!LOCAL && live) out[(size_t)(first + c * CH + t) * ldo + h * dv + e] = o0 + o1;
    }
    __syncthreads();                                             // the buffer is free for the chunk after next
  }
  if (!live) return;
  if (LOCAL) {
    float* L = local + (size_t)tile * seg_elems + (size_t)h * DK * dv;
#pragma unroll
    for (int i = 0; i < DK; ++i) L[(size_t)i * dv + e] = S[i];
  } else if (last) {
#pragma unroll
    for (int i = 0; i < DK; ++i) st[(size_t)i * dv + e] = S[i];
  }
}

template <int DK>
static int launch_segments(const float* proj, int ld, int q_off, int k_off, int v_off, const int* tiles, int n_tiles,
                           int direct, const int* seq_slot, const float* decay, float* state, float* scratch,
                           float* out, int ldo, int H, int dv, int act, cudaStream_t stream) {
  const dim3 grid(n_tiles, H, (dv + 127) / 128), block(128);
  float* local = scratch;
  float* start_copy = scratch ? scratch + (size_t)n_tiles * H * DK * dv : nullptr;
  // whether every piece of a row that is copied starts on a 16-byte boundary
  const int vec = ((size_t)proj & 15) == 0 && ((ld | q_off | k_off | v_off | dv) & 3) == 0;
  if (direct) {
    launch_kernel(lightning_segments_kernel<DK, false, true>, grid, block, 0, stream, proj, ld, q_off, k_off, v_off,
                  tiles, n_tiles, seq_slot, decay, state, local, start_copy, out, ldo, H, dv, act, vec);
    return launch_status();
  }
  if (!scratch) return DLGO_ERR_SIZE;
  launch_kernel(lightning_segments_kernel<DK, true, false>, grid, block, 0, stream, proj, ld, q_off, k_off, v_off, tiles,
                n_tiles, seq_slot, decay, state, local, start_copy, out, ldo, H, dv, act, vec);
  int st = launch_status();
  if (st != DLGO_OK) return st;
  launch_kernel(lightning_segments_kernel<DK, false, false>, grid, block, 0, stream, proj, ld, q_off, k_off, v_off, tiles,
                n_tiles, seq_slot, decay, state, local, start_copy, out, ldo, H, dv, act, vec);
  return launch_status();
}

}  // namespace dlgo

using namespace dlgo;

// 1 if the segment kernels take this qk size (the state's column in registers)
DLGO_EXPORT int dlgo_lightning_segments_takes(int dk) { return dk == 32 || dk == 64 || dk == 128; }

// As dlgo_lightning_scan, with `tiles` [n_tiles, 3] cutting every sequence's tokens into consecutive segments
// (a sequence's segments side by side in the table, in token order).  `direct`: every sequence has exactly one
// segment.  Otherwise `scratch` holds 2 * n_tiles * H * dk * dv floats.
DLGO_EXPORT int dlgo_lightning_segments(const float* proj, int ld, int q_off, int k_off, int v_off, const int* tiles,
                                        int n_tiles, int direct, const int* seq_slot, const float* decay,
                                        float* state, float* scratch, float* out, int ldo, int H, int dk, int dv,
                                        int act, cudaStream_t stream) {
  if (n_tiles <= 0) return DLGO_OK;
  if (H <= 0 || dv <= 0 || n_tiles > 65535 * 32) return DLGO_ERR_SIZE;
#define SEG_ARGS proj, ld, q_off, k_off, v_off, tiles, n_tiles, direct, seq_slot, decay, state, scratch, out, ldo, H, dv, act, stream
  if (dk == 32) return launch_segments<32>(SEG_ARGS);
  if (dk == 64) return launch_segments<64>(SEG_ARGS);
  if (dk == 128) return launch_segments<128>(SEG_ARGS);
  return DLGO_ERR_SIZE;
}

// proj [T, ld] fp32; tiles [n_seqs, 3] (sequence, first packed token, count): one row per sequence of the step;
// state [slots, H, dk, dv] fp32; out [T, ldo] fp32 (heads side by side, dv each)
DLGO_EXPORT int dlgo_lightning_scan(const float* proj, int ld, int q_off, int k_off, int v_off, const int* tiles,
                                    int n_seqs, const int* seq_slot, const float* decay, float* state, float* out,
                                    int ldo, int H, int dk, int dv, int act, cudaStream_t stream) {
  if (n_seqs <= 0) return DLGO_OK;
  if (H <= 0 || dk <= 0 || dv <= 0) return DLGO_ERR_SIZE;
  // as many of a head's value columns per block as keep the block's part of the state within 96 KB
  int dvc = dv;
  while (dvc > 1 && ((size_t)dk * dvc + 2 * (2 * (size_t)dk + dvc)) * sizeof(float) > 96 * 1024) dvc = (dvc + 1) / 2;
  const size_t smem = ((size_t)dk * dvc + 2 * (2 * (size_t)dk + dvc)) * sizeof(float);
  if (smem > 200 * 1024) return DLGO_ERR_SIZE;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(lightning_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int threads = ((dvc + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  if (threads < 64) threads = 64;
  launch_kernel(lightning_scan_kernel, dim3(n_seqs, H, (dv + dvc - 1) / dvc), dim3(threads), smem, stream, proj, ld,
                q_off, k_off, v_off, tiles, seq_slot, decay, state, out, ldo, H, dk, dv, dvc, act);
  return launch_status();
}

// proj [T, ld] fp32, rewritten in place: q heads at q_off, k heads at k_off (H heads of dk numbers each);
// freq [rot / 2] fp32 (may be null with rot == 0); token_pos [T] int32
DLGO_EXPORT int dlgo_rotate_scale(float* proj, int ld, int q_off, int k_off, const float* freq, int rot,
                                  const int* token_pos, int T, int H, int dk, float k_scale, cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (H <= 0 || dk <= 0 || rot < 0 || rot > dk || rot % 2 || (rot > 0 && freq == nullptr)) return DLGO_ERR_SIZE;
  const long long items = (long long)T * 2 * H;
  const long long blocks = (items + RS_WARPS - 1) / RS_WARPS;
  if (blocks > 0x7fffffffLL) return DLGO_ERR_SIZE;
  launch_kernel(rotate_scale_kernel, dim3((unsigned)blocks), dim3(RS_WARPS * 32), 0, stream, proj, ld, q_off, k_off, freq,
                rot, token_pos, T, H, dk, k_scale);
  return launch_status();
}
