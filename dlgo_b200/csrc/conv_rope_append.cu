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
// there, and a second launch (conv_state_keep) stores the step's last ones.  Angles are float(pos) * freq in
// fp32, sincosf; everything here is fp32 until the stores.
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

// The state after the step: a block per sequence of the step (tiles [n, 3]: sequence, its first packed token,
// its token count), a thread per channel, which reads all it needs before it writes.
__global__ void conv_state_keep_kernel(const float* proj, int ld, const float* __restrict__ bias, int n_taps,
                                       float* state, const int* __restrict__ tiles,
                                       const int* __restrict__ seq_slot, int C) {
  pdl_launch_dependents();
  const int seq = tiles[3 * blockIdx.x], tok0 = tiles[3 * blockIdx.x + 1], ntok = tiles[3 * blockIdx.x + 2];
  const int slot = seq_slot[seq];
  const int keep = n_taps - 1;
  pdl_wait();
  float* st = state + (size_t)slot * keep * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
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

DLGO_EXPORT int dlgo_conv_rope_append(const float* proj, int ld, int T, const float* bias, const float* taps,
                                      int n_taps, float* state, const float* freq, int rot, float amplitude,
                                      const int* token_pos, const int* token_seq, const int* seq_slot,
                                      const int* page_table, int max_pages, int page_size, void* q_out, void* kpages,
                                      void* vpages, int dtype, int H, int G, int dk, int dv, int hd, int write_cache,
                                      const int* tiles, int n_tiles, cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || hd < dk || hd < dv || rot < 0 || rot > dk || (rot & 1))
    return DLGO_ERR_SIZE;
  if (n_taps < 1 || n_taps > CONV_MAX_TAPS || (taps == nullptr && n_taps != 1)) return DLGO_ERR_SIZE;
  if (n_taps > 1 && (state == nullptr || tiles == nullptr)) return DLGO_ERR_SIZE;
  if (rot > 0 && freq == nullptr) return DLGO_ERR_SIZE;
  ConvAppendArgs a{proj, ld, T, bias, taps, n_taps, state, freq, rot, amplitude, token_pos, token_seq, seq_slot,
                   page_table, max_pages, page_size, q_out, kpages, vpages, H, G, dk, dv, hd, write_cache};
  const int work = (H + 2 * G) * ((hd + 1) / 2);
  const int threads = work >= 1024 ? 512 : (work >= 256 ? 256 : 128);
  if (dtype == DLGO_F32) launch_kernel(conv_rope_append_kernel<float>, dim3(T), dim3(threads), 0, stream, a);
  else if (dtype == DLGO_BF16) launch_kernel(conv_rope_append_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, a);
  else return DLGO_ERR_DTYPE;
  if (n_taps > 1 && n_tiles > 0) {
    const int C = (H + G) * dk + G * dv;
    launch_kernel(conv_state_keep_kernel, dim3(n_tiles), dim3(C >= 1024 ? 256 : 128), 0, stream, proj, ld, bias, n_taps,
                  state, tiles, seq_slot, C);
  }
  return launch_status();
}
