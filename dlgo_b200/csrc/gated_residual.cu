// A sublayer's way back into the residual stream when its result passes a learned gate, and the weighted
// average over the depth of the model that may follow a layer; with the RMS norm of what comes out for the next
// reader.  One block per token, everything fp32:
//
//   x   <- x + y * sigmoid(g + b)           y: the sublayer's result [T, d] (left zero), g: the gate's logits [T, d]
//                                           from a contraction of their own, b: their bias [d]  (g null: x + y)
//   depth average, if asked for (n_hist > 0): X_(n_hist - 1) = x is stored in the history [n_hist, T, d] and
//   x   <- sum_(j < n_hist) a[j] * X_j      X_0 is the embedding's output, X_j the result of layer j - 1
//   out <- x / sqrt(mean(x^2) + eps) * w    in the run's type, if a norm weight is given
//
// With y null and n_hist = 1 the call stores x as X_0 (a[0] = 1 leaves x as it is).
#include "common.cuh"

namespace dlgo {

template <typename TO>
__global__ void gated_residual_kernel(float* x, float* y, const float* g, int ldg, const float* __restrict__ gate_bias,
                                      float* history, long long hist_stride, int n_hist, const float* __restrict__ avg,
                                      const float* __restrict__ norm_w, float eps, TO* out, int d, int clear_y) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  __shared__ float scale_s;
  const int t = blockIdx.x;
  pdl_wait();
  float* xr = x + (size_t)t * d;
  float* yr = y ? y + (size_t)t * d : nullptr;
  const float* gr = g ? g + (size_t)t * ldg : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = xr[i];
    if (yr != nullptr) {
      float r = yr[i];
      if (gr != nullptr) r *= 1.0f / (1.0f + expf(-(gr[i] + (gate_bias ? gate_bias[i] : 0.f))));
      v += r;
      if (clear_y) yr[i] = 0.f;
    }
    if (n_hist > 0) {
      history[(size_t)(n_hist - 1) * hist_stride + (size_t)t * d + i] = v;
      float m = 0.f;
      for (int j = 0; j < n_hist - 1; ++j) m = fmaf(avg[j], history[(size_t)j * hist_stride + (size_t)t * d + i], m);
      v = fmaf(avg[n_hist - 1], v, m);
    }
    xr[i] = v;
    ss = fmaf(v, v, ss);
  }
  if (norm_w == nullptr) return;
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) scale_s = 1.0f / sqrtf(ss / (float)d + eps);
  __syncthreads();
  const float sc = scale_s;
  TO* o = out + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_float<TO>(xr[i] * sc * norm_w[i]);
}

// logits <- cap * tanh(logits * scale / cap) (cap <= 0: logits * scale), in place
__global__ void scale_softcap_kernel(float* z, long long n, float scale, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = z[i] * scale;
  z[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

}  // namespace dlgo

using namespace dlgo;

DLGO_EXPORT int dlgo_gated_residual(float* x, float* y, const float* g, int ldg, const float* gate_bias, float* history,
                                    long long hist_stride, int n_hist, const float* avg, const float* norm_w, float eps,
                                    void* out, int out_dtype, int T, int d, int clear_y, cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (d <= 0 || n_hist < 0 || (n_hist > 0 && (history == nullptr || avg == nullptr))) return DLGO_ERR_SIZE;
  if (norm_w != nullptr && out == nullptr) return DLGO_ERR_SIZE;
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  if (out_dtype == DLGO_F32)
    launch_kernel(gated_residual_kernel<float>, dim3(T), dim3(threads), 0, stream, x, y, g, ldg, gate_bias, history,
                  hist_stride, n_hist, avg, norm_w, eps, (float*)out, d, clear_y);
  else if (out_dtype == DLGO_BF16)
    launch_kernel(gated_residual_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, x, y, g, ldg, gate_bias,
                  history, hist_stride, n_hist, avg, norm_w, eps, (__nv_bfloat16*)out, d, clear_y);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

DLGO_EXPORT int dlgo_scale_softcap(float* z, long long n, float scale, float cap, cudaStream_t stream) {
  if (n <= 0) return DLGO_OK;
  launch_kernel(scale_softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, z, n, scale, cap);
  return launch_status();
}
