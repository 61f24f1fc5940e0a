// What lies between the q | k | v projection and attention in a mixer whose projections pass through a short
// causal convolution over time: bias, convolution, rotation, cache append.
//
//   u_t   = proj_t + bias                                   (fp32; proj [T, ld] holds q | k | v side by side, heads
//                                                            of dk, dk and dv numbers)
//   y_t   = sum_j taps[c][j] * u_(t - n + 1 + j)            per channel c, n taps, zeros before the sequence's start
//   q, k  : of every head's first `rot` numbers, entries 2i and 2i + 1 turn by the angle pos * freq[i]; cosine and
//           sine are multiplied by `amplitude` (rot = 0: no rotation)
//   q  -> [T, H * hd] in the run's type, k and v -> their page rows [.., G, page, hd]; heads are laid out hd wide
//         with zeros behind their own numbers
//
// The projected values of a sequence's last n - 1 positions are its state ([slots, n - 1, C] fp32, zero when a slot
// is taken, oldest first): a token whose taps reach back past the step's first token of its sequence reads them
// there, and a second launch (conv_state_keep) stores the step's last ones (a step in which every sequence brings
// one token needs none: the token's own thread shifts the state).  Angles are float(pos) * freq in fp32, sincosf;
// everything here is fp32 until the stores.
#include "common.cuh"

namespace dlgo {

constexpr int CONV_MAX_TAPS = 8;

struct ConvAppendArgs {
  const float* proj;         // [T, ld]
  int ld, T;
  const float* bias;         // [C] or null
  const float* taps;         // [C, n] or null (n = 1 and no taps: no convolution)
  int n_taps;
  const float* state;        // [slots, n - 1, C]
  const float* freq;         // [rot / 2]
  int rot;
  float amplitude;
  const int* token_pos;
  const int* token_seq;
  const int* seq_slot;
  const int* page_table;
  int max_pages, page_size;
  void* q_out;               // [T, H * hd]
  void* kpages;
  void* vpages;
  int H, G, dk, dv, hd;
  int write_cache;
  int keep_alone;            // a token that is its sequence's only one in the step shifts the state itself
  int clear_proj;            // every sequence brings one token, and proj is a sum that must be zero again afterwards
};

// a block per token; a thread per pair of neighbouring numbers of a head (the last of an odd head alone)
template <typename T>
__global__ void conv_rope_append_kernel(ConvAppendArgs a) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int C = (a.H + a.G) * a.dk + a.G * a.dv;
  const int seq = a.token_seq[t];
  const int pos = a.token_pos[t];
  const int slot = a.seq_slot[seq];
  // rows of the same sequence directly before this one in the step (as many as the taps can reach)
  int n_in = 0;
  while (n_in < a.n_taps - 1 && t - n_in - 1 >= 0 && a.token_seq[t - n_in - 1] == seq) ++n_in;
  const int page = a.page_table[(size_t)slot * a.max_pages + pos / a.page_size];
  const int n_heads = a.H + 2 * a.G;
  const int pairs = (a.hd + 1) / 2;
  pdl_wait();
  const float* st = a.state + (size_t)slot * (a.n_taps - 1) * C;
  for (int idx = threadIdx.x; idx < n_heads * pairs; idx += blockDim.x) {
    const int head = idx / pairs, e = (idx - head * pairs) * 2;
    // which of q, k, v the head belongs to; its own size and where its channels start
    int kind, hh, width, c0;
    if (head < a.H) { kind = 0; hh = head; width = a.dk; c0 = hh * a.dk; }
    else if (head < a.H + a.G) { kind = 1; hh = head - a.H; width = a.dk; c0 = a.H * a.dk + hh * a.dk; }
    else { kind = 2; hh = head - a.H - a.G; width = a.dv; c0 = (a.H + a.G) * a.dk + hh * a.dv; }
    float y[2] = {0.f, 0.f};
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      if (e + s >= width) continue;
      const int c = c0 + e + s;
      const float b = a.bias ? a.bias[c] : 0.f;
      if (a.taps == nullptr) {
        y[s] = a.proj[(size_t)t * a.ld + c] + b;
        continue;
      }
      float acc = 0.f;
      for (int j = 0; j < a.n_taps; ++j) {
        const int back = a.n_taps - 1 - j;        // how many positions before this token
        float u;
        if (back <= n_in) u = a.proj[(size_t)(t - back) * a.ld + c] + b;
        else u = st[(size_t)(a.n_taps - 1 - (back - n_in)) * C + c];
        acc = fmaf(a.taps[(size_t)c * a.n_taps + j], u, acc);
      }
      y[s] = acc;
    }
    if (kind < 2 && e < a.rot) {
      float sn, cs;
      sincosf((float)pos * a.freq[e >> 1], &sn, &cs);
      sn *= a.amplitude;
      cs *= a.amplitude;
      const float u = y[0], v = y[1];
      y[0] = u * cs - v * sn;
      y[1] = v * cs + u * sn;
    }
    T* dst = nullptr;
    if (kind == 0) {
      dst = (T*)a.q_out + ((size_t)t * a.H + hh) * a.hd;
    } else if (a.write_cache && page >= 0) {
      T* pages = (T*)(kind == 1 ? a.kpages : a.vpages);
      dst = pages + (((size_t)page * a.G + hh) * a.page_size + pos % a.page_size) * a.hd;
    }
    if (dst == nullptr) continue;
    dst[e] = from_float<T>(e < width ? y[0] : 0.f);
    if (e + 1 < a.hd) dst[e + 1] = from_float<T>(e + 1 < width ? y[1] : 0.f);
  }
}

// The same for even head sizes and a known number of taps (NT <= 4): a thread's two channels travel as one 8-byte
// piece, and the NT rows it needs (of the step, or of the state) and its taps are all fetched before the first use.
// With `keep_alone` a token that is the only one of its sequence in the step (decoding) writes the shifted state
// itself: its thread has just read every entry of its two channels, and nobody else touches that sequence's row.
template <typename T, int NT>
__global__ void __launch_bounds__(256) conv_rope_append_pairs_kernel(ConvAppendArgs a) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int C = (a.H + a.G) * a.dk + a.G * a.dv;
  const int seq = a.token_seq[t];
  const int pos = a.token_pos[t];
  const int slot = a.seq_slot[seq];
  int n_in = 0;
  while (n_in < NT - 1 && t - n_in - 1 >= 0 && a.token_seq[t - n_in - 1] == seq) ++n_in;
  const int page = a.page_table[(size_t)slot * a.max_pages + pos / a.page_size];
  const int n_heads = a.H + 2 * a.G;
  const int pairs = a.hd >> 1;
  const bool alone = a.keep_alone && NT > 1 && n_in == 0 && (t + 1 >= a.T || a.token_seq[t + 1] != seq);
  pdl_wait();
  float* st = const_cast<float*>(a.state) + (size_t)slot * (NT - 1) * C;
  for (int idx = threadIdx.x; idx < n_heads * pairs; idx += blockDim.x) {
    const int head = idx / pairs, e = (idx - head * pairs) * 2;
    int kind, hh, width, c0;
    if (head < a.H) { kind = 0; hh = head; width = a.dk; c0 = hh * a.dk; }
    else if (head < a.H + a.G) { kind = 1; hh = head - a.H; width = a.dk; c0 = a.H * a.dk + hh * a.dk; }
    else { kind = 2; hh = head - a.H - a.G; width = a.dv; c0 = (a.H + a.G) * a.dk + hh * a.dv; }
    float2 y = make_float2(0.f, 0.f);
    if (e < width) {
      const int c = c0 + e;
      const float2 b = a.bias ? __ldg(reinterpret_cast<const float2*>(a.bias + c)) : make_float2(0.f, 0.f);
      float2 u[NT], w[NT];       // w: taps of channel c (NT numbers), then of channel c + 1, as NT pieces of two
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int back = NT - 1 - j;
        if (back <= n_in) {
          u[j] = *reinterpret_cast<const float2*>(a.proj + (size_t)(t - back) * a.ld + c);
          if (a.clear_proj) *reinterpret_cast<float2*>(const_cast<float*>(a.proj) + (size_t)t * a.ld + c) = make_float2(0.f, 0.f);
          u[j].x += b.x;
          u[j].y += b.y;
        } else {
          u[j] = *reinterpret_cast<const float2*>(st + (size_t)(NT - 1 - (back - n_in)) * C + c);
        }
        if (NT > 1) w[j] = __ldg(reinterpret_cast<const float2*>(a.taps + (size_t)c * NT) + j);
      }
      if (alone) {
#pragma unroll
        for (int j = 0; j + 1 < NT; ++j) *reinterpret_cast<float2*>(st + (size_t)j * C + c) = u[j + 1];
      }
      if (NT == 1 && a.taps == nullptr) {
        y = u[0];
      } else if (NT == 1) {
        y = make_float2(a.taps[c] * u[0].x, a.taps[c + 1] * u[0].y);
      } else {
        const float* wf = reinterpret_cast<const float*>(w);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          y.x = fmaf(wf[j], u[j].x, y.x);
          y.y = fmaf(wf[NT + j], u[j].y, y.y);
        }
      }
      if (kind < 2 && e < a.rot) {
        float sn, cs;
        sincosf((float)pos * a.freq[e >> 1], &sn, &cs);
        sn *= a.amplitude;
        cs *= a.amplitude;
        const float p0 = y.x, p1 = y.y;
        y.x = p0 * cs - p1 * sn;
        y.y = p1 * cs + p0 * sn;
      }
    }
    T* dst = nullptr;
    if (kind == 0) {
      dst = (T*)a.q_out + ((size_t)t * a.H + hh) * a.hd;
    } else if (a.write_cache && page >= 0) {
      T* pages = (T*)(kind == 1 ? a.kpages : a.vpages);
      dst = pages + (((size_t)page * a.G + hh) * a.page_size + pos % a.page_size) * a.hd;
    }
    if (dst == nullptr) continue;
    if (sizeof(T) == 2) *reinterpret_cast<__nv_bfloat162*>(dst + e) = __floats2bfloat162_rn(y.x, y.y);
    else *reinterpret_cast<float2*>(dst + e) = y;
  }
}

// Many tokens (prompts): a block walks CT_TOKENS consecutive rows, a thread keeping its two channels' last NT - 1
// values in registers, so that a row of proj is read once (not once per tap) and taps, bias and the head's place are
// looked up once per block.  All of the tile's own values are fetched before the walk begins.  The state is left to
// the second launch.
constexpr int CT_TOKENS = 8;

template <typename T, int NT>
__global__ void __launch_bounds__(128) conv_rope_append_tiles_kernel(ConvAppendArgs a) {
  pdl_launch_dependents();
  const int C = (a.H + a.G) * a.dk + a.G * a.dv;
  const int pairs = a.hd >> 1;
  const int idx = blockIdx.y * blockDim.x + threadIdx.x;
  const int t0 = blockIdx.x * CT_TOKENS;
  const int nt = min(CT_TOKENS, a.T - t0);
  if (idx >= (a.H + 2 * a.G) * pairs) return;
  const int head = idx / pairs, e = (idx - head * pairs) * 2;
  int kind, hh, width, c0;
  if (head < a.H) { kind = 0; hh = head; width = a.dk; c0 = hh * a.dk; }
  else if (head < a.H + a.G) { kind = 1; hh = head - a.H; width = a.dk; c0 = a.H * a.dk + hh * a.dk; }
  else { kind = 2; hh = head - a.H - a.G; width = a.dv; c0 = (a.H + a.G) * a.dk + hh * a.dv; }
  const bool live = e < width;                 // (else: zeros behind the head's own numbers)
  const int c = c0 + (live ? e : 0);
  const float2 b = (live && a.bias) ? __ldg(reinterpret_cast<const float2*>(a.bias + c)) : make_float2(0.f, 0.f);
  float w0[NT], w1[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    w0[j] = (live && a.taps) ? __ldg(a.taps + (size_t)c * NT + j) : (j == NT - 1 ? 1.f : 0.f);
    w1[j] = (live && a.taps) ? __ldg(a.taps + (size_t)(c + 1) * NT + j) : (j == NT - 1 ? 1.f : 0.f);
  }
  const bool turns = kind < 2 && live && e < a.rot;
  const float f = turns ? a.freq[e >> 1] : 0.f;
  // the tile's sequences and positions: the step's own inputs, fetched before the wait
  int seqs[CT_TOKENS], poss[CT_TOKENS];
#pragma unroll
  for (int i = 0; i < CT_TOKENS; ++i) {
    seqs[i] = i < nt ? a.token_seq[t0 + i] : -1;
    poss[i] = i < nt ? a.token_pos[t0 + i] : 0;
  }
  pdl_wait();
  float2 cur[CT_TOKENS];
#pragma unroll
  for (int i = 0; i < CT_TOKENS; ++i) {
    cur[i] = make_float2(0.f, 0.f);
    if (live && i < nt) {
      cur[i] = *reinterpret_cast<const float2*>(a.proj + (size_t)(t0 + i) * a.ld + c);
      cur[i].x += b.x;
      cur[i].y += b.y;
    }
  }
  float2 win[NT > 1 ? NT - 1 : 1];
  int prev_seq = -1, slot = 0;
#pragma unroll
  for (int i = 0; i < CT_TOKENS; ++i) {
    if (i >= nt) break;
    const int t = t0 + i;
    const int seq = seqs[i];
    const int pos = poss[i];
    if (seq != prev_seq) {
      // the sequence's rows before this one: of this step (as far as the taps reach), else of its state
      slot = a.seq_slot[seq];
      prev_seq = seq;
      if (NT > 1 && live) {
        int n_in = 0;
        while (n_in < NT - 1 && t - n_in - 1 >= 0 && a.token_seq[t - n_in - 1] == seq) ++n_in;
        const float* st = a.state + (size_t)slot * (NT - 1) * C;
#pragma unroll
        for (int j = 0; j < NT - 1; ++j) {
          const int back = NT - 1 - j;
          if (back <= n_in) {
            win[j] = *reinterpret_cast<const float2*>(a.proj + (size_t)(t - back) * a.ld + c);
            win[j].x += b.x;
            win[j].y += b.y;
          } else {
            win[j] = *reinterpret_cast<const float2*>(st + (size_t)(NT - 1 - (back - n_in)) * C + c);
          }
        }
      }
    }
    float2 y = make_float2(w0[NT - 1] * cur[i].x, w1[NT - 1] * cur[i].y);
    if (NT > 1) {
#pragma unroll
      for (int j = 0; j < NT - 1; ++j) {
        y.x = fmaf(w0[j], win[j].x, y.x);
        y.y = fmaf(w1[j], win[j].y, y.y);
      }
#pragma unroll
      for (int j = 0; j + 1 < NT - 1; ++j) win[j] = win[j + 1];
      win[NT - 2 >= 0 ? NT - 2 : 0] = cur[i];
    }
    if (!live) y = make_float2(0.f, 0.f);
    if (turns) {
      float sn, cs;
      sincosf((float)pos * f, &sn, &cs);
      sn *= a.amplitude;
      cs *= a.amplitude;
      const float p0 = y.x, p1 = y.y;
      y.x = p0 * cs - p1 * sn;
      y.y = p1 * cs + p0 * sn;
    }
    T* dst = nullptr;
    if (kind == 0) {
      dst = (T*)a.q_out + ((size_t)t * a.H + hh) * a.hd;
    } else if (a.write_cache) {
      const int page = a.page_table[(size_t)slot * a.max_pages + pos / a.page_size];
      T* pages = (T*)(kind == 1 ? a.kpages : a.vpages);
      if (page >= 0) dst = pages + (((size_t)page * a.G + hh) * a.page_size + pos % a.page_size) * a.hd;
    }
    if (dst == nullptr) continue;
    if (sizeof(T) == 2) *reinterpret_cast<__nv_bfloat162*>(dst + e) = __floats2bfloat162_rn(y.x, y.y);
    else *reinterpret_cast<float2*>(dst + e) = y;
  }
}

// The state after the step: a block per sequence of the step (tiles [n, 3]: sequence, its first packed token,
// its token count), a thread per channel, which reads all it needs before it writes.
__global__ void conv_state_keep_kernel(const float* proj, int ld, const float* __restrict__ bias, int n_taps,
                                       float* state, const int* __restrict__ tiles,
                                       const int* __restrict__ seq_slot, int C, int skip_alone) {
  pdl_launch_dependents();
  const int seq = tiles[3 * blockIdx.x], tok0 = tiles[3 * blockIdx.x + 1], ntok = tiles[3 * blockIdx.x + 2];
  const int slot = seq_slot[seq];
  const int keep = n_taps - 1;
  pdl_wait();
  if (skip_alone && ntok == 1) return;       // (its own token has shifted the state)
  float* st = state + (size_t)slot * keep * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float v[CONV_MAX_TAPS];
    const float b = bias ? bias[c] : 0.f;
    for (int k = 0; k < keep; ++k) {
      // entry k of the new state is the position keep - k before the sequence's new end
      const int back = keep - k;
      v[k] = back <= ntok ? proj[(size_t)(tok0 + ntok - back) * ld + c] + b : st[(size_t)(k + ntok) * C + c];
    }
    for (int k = 0; k < keep; ++k) st[(size_t)k * C + c] = v[k];
  }
}

}  // namespace dlgo

using namespace dlgo;

// Whether, for these sizes, a step whose sequences bring one token each can take proj as a sum to be cleared.
DLGO_EXPORT int dlgo_conv_rope_append_clears(int dk, int dv, int hd, int ld, int n_taps) {
  return !(dk & 1) && !(dv & 1) && !(hd & 1) && !(ld & 1) && n_taps <= 4;
}

DLGO_EXPORT int dlgo_conv_rope_append(const float* proj, int ld, int T, const float* bias, const float* taps,
                                      int n_taps, float* state, const float* freq, int rot, float amplitude,
                                      const int* token_pos, const int* token_seq, const int* seq_slot,
                                      const int* page_table, int max_pages, int page_size, void* q_out, void* kpages,
                                      void* vpages, int dtype, int H, int G, int dk, int dv, int hd, int write_cache,
                                      const int* tiles, int n_tiles, int all_alone, int clear_proj,
                                      cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || hd < dk || hd < dv || rot < 0 || rot > dk || (rot & 1))
    return DLGO_ERR_SIZE;
  if (n_taps < 1 || n_taps > CONV_MAX_TAPS || (taps == nullptr && n_taps != 1)) return DLGO_ERR_SIZE;
  if (n_taps > 1 && (state == nullptr || tiles == nullptr)) return DLGO_ERR_SIZE;
  if (rot > 0 && freq == nullptr) return DLGO_ERR_SIZE;
  ConvAppendArgs a{proj, ld, T, bias, taps, n_taps, state, freq, rot, amplitude, token_pos, token_seq, seq_slot,
                   page_table, max_pages, page_size, q_out, kpages, vpages, H, G, dk, dv, hd, write_cache, 0, 0};
  const int work = (H + 2 * G) * ((hd + 1) / 2);
  const int threads = work >= 1024 ? 512 : (work >= 256 ? 256 : 128);
  if (dtype != DLGO_F32 && dtype != DLGO_BF16) return DLGO_ERR_DTYPE;
  const bool even = !(dk & 1) && !(dv & 1) && !(hd & 1) && !(ld & 1) && ((uintptr_t)proj & 7) == 0 &&
                    ((uintptr_t)state & 7) == 0 && ((uintptr_t)bias & 7) == 0 && ((uintptr_t)taps & 7) == 0 &&
                    ((uintptr_t)q_out & 7) == 0 && ((uintptr_t)kpages & 7) == 0 && ((uintptr_t)vpages & 7) == 0;
  // (only the kernel for even sizes and few taps clears proj: dlgo_conv_rope_append_clears says whether it runs)
  if (clear_proj && !(all_alone && even && n_taps <= 4)) return DLGO_ERR_SIZE;
  bool kept = false;      // whether tokens alone in their sequence keep the state themselves
  if (even && n_taps <= 4 && T > 64 && !all_alone) {
    // prompts: tiles of tokens, the state left to the second launch
    const dim3 grid((T + CT_TOKENS - 1) / CT_TOKENS, ((H + 2 * G) * (hd >> 1) + 127) / 128);
#define DLGO_CONV_TILES(NT)                                                                                            \
  do {                                                                                                                 \
    if (dtype == DLGO_F32) launch_kernel(conv_rope_append_tiles_kernel<float, NT>, grid, dim3(128), 0, stream, a);     \
    else launch_kernel(conv_rope_append_tiles_kernel<__nv_bfloat16, NT>, grid, dim3(128), 0, stream, a);               \
  } while (0)
    if (n_taps == 1) DLGO_CONV_TILES(1);
    else if (n_taps == 2) DLGO_CONV_TILES(2);
    else if (n_taps == 3) DLGO_CONV_TILES(3);
    else DLGO_CONV_TILES(4);
#undef DLGO_CONV_TILES
  } else if (even && n_taps <= 4) {
    const int th = work >= 256 ? 256 : 128;
    a.keep_alone = kept = n_taps > 1;
    a.clear_proj = clear_proj && all_alone;
#define DLGO_CONV(NT)                                                                                                  \
  do {                                                                                                                 \
    if (dtype == DLGO_F32) launch_kernel(conv_rope_append_pairs_kernel<float, NT>, dim3(T), dim3(th), 0, stream, a);   \
    else launch_kernel(conv_rope_append_pairs_kernel<__nv_bfloat16, NT>, dim3(T), dim3(th), 0, stream, a);             \
  } while (0)
    if (n_taps == 1) DLGO_CONV(1);
    else if (n_taps == 2) DLGO_CONV(2);
    else if (n_taps == 3) DLGO_CONV(3);
    else DLGO_CONV(4);
#undef DLGO_CONV
  } else if (dtype == DLGO_F32) {
    launch_kernel(conv_rope_append_kernel<float>, dim3(T), dim3(threads), 0, stream, a);
  } else {
    launch_kernel(conv_rope_append_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, a);
  }
  // `all_alone` (the caller's word that every sequence brings one token): nothing is left for the second launch
  if (n_taps > 1 && n_tiles > 0 && !(kept && all_alone)) {
    const int C = (H + G) * dk + G * dv;
    launch_kernel(conv_state_keep_kernel, dim3(n_tiles, (C + 255) / 256), dim3(256), 0, stream, proj, ld, bias, n_taps,
                  state, tiles, seq_slot, C, kept ? 1 : 0);
  }
  return launch_status();
}
