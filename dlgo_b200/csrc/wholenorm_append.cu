// Queries and keys normed over their WHOLE projection (all heads at once), the append of this step's keys and
// values to the paged cache, and one gate per query head, in one pass over the fp32 result of the q|k|v|gate
// projection; and the multiplication of attention's result by those gates.
//
// proj[T, ld] (fp32): Hq * dk query numbers, then Hkv * dk key numbers, then Hkv * dv value numbers, then
// (`has_gate`) Hq gate logits.
//
//   q <- q / sqrt(mean over all Hq * dk numbers of q^2 + eps) * w_q        (w_q has Hq * dk numbers; null: no norm)
//   k <- k / sqrt(mean over all Hkv * dk numbers of k^2 + eps) * w_k
//   gate[h] = sigmoid(logit[h]) * gate_scale
//
// Heads are laid out `hd` numbers wide (hd >= dk, hd >= dv) with zeros behind a head's own numbers, so that keys
// and values share one page shape and the framework's attention kernels, which take one head size, run on them:
// zeros add nothing to a score and give zeros in the result that the output projection's zero columns ignore.
// q goes to q_out[T, Hq * hd] in the run's type; k and v go to the page of the token's position:
// pages[page_table[slot][pos / PS]][kv_head][pos % PS][:].  `clear`: zeros are left in proj.
// Statistics and norm are fp32; one rounding at the final store.
#include "common.cuh"

namespace dlgo {

// Set when a token's position had no page in the table (-1): the append is skipped.
__device__ int g_wholenorm_append_error = 0;

template <typename T>
__global__ void __launch_bounds__(128)
wholenorm_append_kernel(float* proj, int ld, const float* __restrict__ w_q, const float* __restrict__ w_k,
                        float eps, const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                        const int* __restrict__ seq_slot, const int* __restrict__ page_table, int max_pages,
                        T* kpages, T* vpages, T* q_out,
                        float* gate_out, int Hq, int Hkv, int dk, int dv, int hd, int page_size,
                        int has_gate, float gate_scale, int write_cache, int clear) {
  __shared__ float red[32];
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int pos = token_pos[t];              // the step's own inputs: in place before the step's first kernel starts
  long long row_base = -1;                   // first element of this position's row of kv head 0 in a page
  if (write_cache) {
    const int slot = seq_slot[token_seq[t]];
    const int page = page_table[(size_t)slot * max_pages + pos / page_size];
    if (page < 0) {
      if (threadIdx.x == 0) atomicExch(&g_wholenorm_append_error, 1);
    } else {
      row_base = ((long long)page * Hkv * page_size + (pos % page_size)) * hd;
    }
  }
  const int nq = Hq * dk, nk = Hkv * dk, nv = Hkv * dv;
  pdl_wait();
  float* src = proj + (size_t)t * ld;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nq; i += blockDim.x) sq = fmaf(src[i], src[i], sq);
  for (int i = threadIdx.x; i < nk; i += blockDim.x) sk = fmaf(src[nq + i], src[nq + i], sk);
  sq = block_sum(sq, red);
  sk = block_sum(sk, red);
  const float rq = w_q != nullptr ? 1.0f / sqrtf(sq / (float)nq + eps) : 1.0f;
  const float rk = w_k != nullptr ? 1.0f / sqrtf(sk / (float)nk + eps) : 1.0f;
  for (int i = threadIdx.x; i < Hq * hd; i += blockDim.x) {
    const int h = i / hd, c = i - h * hd;
    float val = 0.f;
    if (c < dk) val = src[h * dk + c] * rq * (w_q != nullptr ? w_q[h * dk + c] : 1.0f);
    q_out[(size_t)t * Hq * hd + i] = from_float<T>(val);
  }
  if (row_base >= 0) {
    for (int i = threadIdx.x; i < Hkv * hd; i += blockDim.x) {
      const int g = i / hd, c = i - g * hd;
      float kval = 0.f, vval = 0.f;
      if (c < dk) kval = src[nq + g * dk + c] * rk * (w_k != nullptr ? w_k[g * dk + c] : 1.0f);
      if (c < dv) vval = src[nq + nk + g * dv + c];
      const size_t at = (size_t)row_base + (size_t)g * page_size * hd + c;
      kpages[at] = from_float<T>(kval);
      vpages[at] = from_float<T>(vval);
    }
  }
  if (has_gate)
    for (int h = threadIdx.x; h < Hq; h += blockDim.x)
      gate_out[(size_t)t * Hq + h] = gate_scale / (1.0f + expf(-src[nq + nk + nv + h]));
  if (clear) {
    __syncthreads();             // every read of the row is done
    const int n = nq + nk + nv + (has_gate ? Hq : 0);
    for (int i = threadIdx.x; i < n; i += blockDim.x) src[i] = 0.f;
  }
}

// a[t, h, :] *= gate[t, h]   (a in the run's type, heads of hd numbers; the product is formed in fp32)
template <typename T>
__global__ void __launch_bounds__(256)
scale_heads_kernel(T* a, const float* gate, long long total, int hd) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    a[i] = from_float<T>(to_float(a[i]) * gate[i / hd]);
}

template <typename T>
int launch_wholenorm_append(float* proj, int ld, const float* w_q, const float* w_k, float eps, const int* token_pos,
                            const int* token_seq, const int* seq_slot, const int* page_table, int max_pages,
                            void* kpages, void* vpages, void* q_out, float* gate_out, int T_tokens, int Hq, int Hkv,
                            int dk, int dv, int hd, int page_size, int has_gate, float gate_scale, int write_cache,
                            int clear, cudaStream_t stream) {
  launch_kernel(wholenorm_append_kernel<T>, dim3(T_tokens), dim3(128), 0, stream, proj, ld, w_q, w_k, eps, token_pos,
                token_seq, seq_slot, page_table, max_pages, (T*)kpages, (T*)vpages, (T*)q_out, gate_out, Hq, Hkv, dk, dv,
                hd, page_size, has_gate, gate_scale, write_cache, clear);
  return launch_status();
}

}  // namespace dlgo

DLGO_EXPORT int dlgo_wholenorm_append(float* proj, int ld, const float* w_q, const float* w_k, float eps,
                                      const int* token_pos, const int* token_seq, const int* seq_slot,
                                      const int* page_table, int max_pages, void* kpages, void* vpages, void* q_out,
                                      float* gate_out, int dtype, int T, int Hq, int Hkv, int dk, int dv, int hd,
                                      int page_size, int has_gate, float gate_scale, int write_cache, int clear,
                                      cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (Hq <= 0 || Hkv <= 0 || dk <= 0 || dv <= 0 || hd < dk || hd < dv) return DLGO_ERR_SIZE;
  if (ld < Hq * dk + Hkv * (dk + dv) + (has_gate ? Hq : 0)) return DLGO_ERR_SIZE;
  if (has_gate && gate_out == nullptr) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32)
    return dlgo::launch_wholenorm_append<float>(proj, ld, w_q, w_k, eps, token_pos, token_seq, seq_slot, page_table,
                                                max_pages, kpages, vpages, q_out, gate_out, T, Hq, Hkv, dk, dv, hd,
                                                page_size, has_gate, gate_scale, write_cache, clear, stream);
  if (dtype == DLGO_BF16)
    return dlgo::launch_wholenorm_append<__nv_bfloat16>(proj, ld, w_q, w_k, eps, token_pos, token_seq, seq_slot,
                                                        page_table, max_pages, kpages, vpages, q_out, gate_out, T, Hq,
                                                        Hkv, dk, dv, hd, page_size, has_gate, gate_scale, write_cache,
                                                        clear, stream);
  return DLGO_ERR_DTYPE;
}

// a [T, H * hd] in `dtype` (contiguous), gate [T, H] fp32
DLGO_EXPORT int dlgo_scale_heads(void* a, const float* gate, int dtype, int T, int H, int hd, cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (H <= 0 || hd <= 0) return DLGO_ERR_SIZE;
  const long long total = (long long)T * H * hd;
  const long long want = (total + 255) / 256;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == DLGO_F32)
    dlgo::launch_kernel(dlgo::scale_heads_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)a, gate, total, hd);
  else if (dtype == DLGO_BF16)
    dlgo::launch_kernel(dlgo::scale_heads_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)a,
                        gate, total, hd);
  else
    return DLGO_ERR_DTYPE;
  return dlgo::launch_status();
}

// The error word (1: a position had no page), cleared by the read.
DLGO_EXPORT int dlgo_wholenorm_append_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, dlgo::g_wholenorm_append_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(dlgo::g_wholenorm_append_error, &zero, sizeof(int));
  return v;
}
