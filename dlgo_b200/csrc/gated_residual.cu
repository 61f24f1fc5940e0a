// A sublayer's way back into the residual stream when its result passes a learned gate, and the weighted
// average over the depth of the model that may follow a layer; with the RMS norm of what comes out for the next
// reader.  One block per token, everything fp32:
//
//   x   <- x + (y + c) * sigmoid(g + b)     y: the sublayer's result [T, d] (left zero), c: a bias [d] that the
//                                           sublayer left to this pass (or null), g: the gate's logits [T, d] from a
//                                           contraction of their own (left zero if asked: a sum that the contraction
//                                           adds into), b: their bias [d]  (g null: x + y + c)
//   depth average, if asked for (n_hist > 0): X_(n_hist - 1) = x is stored in the history [n_hist, T, d] and
//   x   <- sum_(j < n_hist) a[j] * X_j      X_0 is the embedding's output, X_j the result of layer j - 1
//   out <- x / sqrt(mean(x^2) + eps) * w    in the run's type, if a norm weight is given
//
// With y null and n_hist = 1 the call stores x as X_0 (a[0] = 1 leaves x as it is).
#include "common.cuh"

namespace dlgo {

template <typename TO>
__global__ void gated_residual_kernel(float* x, float* y, const float* __restrict__ y_bias, const float* g, int ldg,
                                      const float* __restrict__ gate_bias,
                                      float* history, long long hist_stride, int n_hist, const float* __restrict__ avg,
                                      const float* __restrict__ norm_w, float eps, TO* out, int d, int clear_y, int clear_g) {
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
      float r = yr[i] + (y_bias ? y_bias[i] : 0.f);
      if (gr != nullptr) {
        r *= 1.0f / (1.0f + expf(-(gr[i] + (gate_bias ? gate_bias[i] : 0.f))));
        if (clear_g) const_cast<float*>(gr)[i] = 0.f;
      }
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

// The same with a row in registers: a thread owns NV pieces of four neighbouring numbers (d a multiple of 4, at most
// 4 * NV * blockDim numbers, 16-byte aligned rows); every load of a piece is issued before its first use, and the
// norm's output is written from the registers.
template <typename TO> __device__ __forceinline__ void store4(TO* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

__device__ __forceinline__ float sigmoid_of(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename TO, int NV>
__global__ void __launch_bounds__(256)
gated_residual_rows_kernel(float* x, float* y, const float* __restrict__ y_bias, const float* g, int ldg,
                           const float* __restrict__ gate_bias,
                           float* history, long long hist_stride, int n_hist, const float* __restrict__ avg,
                           const float* __restrict__ norm_w, float eps, TO* out, int d, int clear_y, int clear_g) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  __shared__ float scale_s;
  const int t = blockIdx.x;
  const int n4 = d >> 2;
  float4 gb[NV], nw[NV], yb[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
    gb[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    nw[k] = gb[k];
    yb[k] = gb[k];
    if (i < n4) {
      if (y_bias != nullptr) yb[k] = __ldg(reinterpret_cast<const float4*>(y_bias) + i);
      if (gate_bias != nullptr && g != nullptr) gb[k] = __ldg(reinterpret_cast<const float4*>(gate_bias) + i);
      if (norm_w != nullptr) nw[k] = __ldg(reinterpret_cast<const float4*>(norm_w) + i);
    }
  }
  pdl_wait();
  float4* xr = reinterpret_cast<float4*>(x + (size_t)t * d);
  float4* yr = y ? reinterpret_cast<float4*>(y + (size_t)t * d) : nullptr;
  const float4* gr = g ? reinterpret_cast<const float4*>(g + (size_t)t * ldg) : nullptr;
  float4 v[NV], r[NV], gl[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      v[k] = xr[i];
      if (yr != nullptr) r[k] = yr[i];
      if (gr != nullptr) {
        gl[k] = gr[i];
        if (clear_g) const_cast<float4*>(gr)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i >= n4) continue;
    if (yr != nullptr) {
      r[k].x += yb[k].x; r[k].y += yb[k].y; r[k].z += yb[k].z; r[k].w += yb[k].w;
      if (gr != nullptr) {
        r[k].x *= sigmoid_of(gl[k].x + gb[k].x);
        r[k].y *= sigmoid_of(gl[k].y + gb[k].y);
        r[k].z *= sigmoid_of(gl[k].z + gb[k].z);
        r[k].w *= sigmoid_of(gl[k].w + gb[k].w);
      }
      v[k].x += r[k].x; v[k].y += r[k].y; v[k].z += r[k].z; v[k].w += r[k].w;
      if (clear_y) yr[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (n_hist > 0) {
      float4* hrow = reinterpret_cast<float4*>(history + (size_t)t * d);
      const size_t hs4 = (size_t)(hist_stride >> 2);
      hrow[(size_t)(n_hist - 1) * hs4 + i] = v[k];
      float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < n_hist - 1; ++j) {
        const float a = avg[j];
        const float4 h = hrow[(size_t)j * hs4 + i];
        m.x = fmaf(a, h.x, m.x); m.y = fmaf(a, h.y, m.y); m.z = fmaf(a, h.z, m.z); m.w = fmaf(a, h.w, m.w);
      }
      const float a = avg[n_hist - 1];
      v[k] = make_float4(fmaf(a, v[k].x, m.x), fmaf(a, v[k].y, m.y), fmaf(a, v[k].z, m.z), fmaf(a, v[k].w, m.w));
    }
    xr[i] = v[k];
    ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss); ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss);
  }
  if (norm_w == nullptr) return;
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) scale_s = 1.0f / sqrtf(ss / (float)d + eps);
  __syncthreads();
  const float sc = scale_s;
  TO* o = out + (size_t)t * d;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4)
      store4<TO>(o + 4 * (size_t)i, make_float4(v[k].x * sc * nw[k].x, v[k].y * sc * nw[k].y, v[k].z * sc * nw[k].z,
                                                  v[k].w * sc * nw[k].w));
  }
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

DLGO_EXPORT int dlgo_gated_residual(float* x, float* y, const float* y_bias, const float* g, int ldg,
                                    const float* gate_bias, float* history,
                                    long long hist_stride, int n_hist, const float* avg, const float* norm_w, float eps,
                                    void* out, int out_dtype, int T, int d, int clear_y, int clear_g,
                                    cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (d <= 0 || n_hist < 0 || (n_hist > 0 && (history == nullptr || avg == nullptr))) return DLGO_ERR_SIZE;
  if (norm_w != nullptr && out == nullptr) return DLGO_ERR_SIZE;
  const bool rows16 = ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)g & 15) == 0 &&
                      ((uintptr_t)history & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)gate_bias & 15) == 0 &&
                      ((uintptr_t)norm_w & 15) == 0 && ((uintptr_t)y_bias & 15) == 0 && (ldg & 3) == 0 && (hist_stride & 3) == 0;
  if ((d & 3) == 0 && d <= 8192 && rows16) {
#define DLGO_GR(NV)                                                                                                  \
  do {                                                                                                               \
    if (out_dtype == DLGO_F32)                                                                                       \
      launch_kernel(gated_residual_rows_kernel<float, NV>, dim3(T), dim3(256), 0, stream, x, y, y_bias, g, ldg, gate_bias,   \
                    history, hist_stride, n_hist, avg, norm_w, eps, (float*)out, d, clear_y, clear_g);                        \
    else if (out_dtype == DLGO_BF16)                                                                                 \
      launch_kernel(gated_residual_rows_kernel<__nv_bfloat16, NV>, dim3(T), dim3(256), 0, stream, x, y, y_bias, g, ldg, \
                    gate_bias, history, hist_stride, n_hist, avg, norm_w, eps, (__nv_bfloat16*)out, d, clear_y, clear_g);     \
    else                                                                                                             \
      return DLGO_ERR_DTYPE;                                                                                         \
  } while (0)
    if (d <= 1024) DLGO_GR(1);
    else if (d <= 2048) DLGO_GR(2);
    else if (d <= 4096) DLGO_GR(4);
    else DLGO_GR(8);
#undef DLGO_GR
    return launch_status();
  }
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  if (out_dtype == DLGO_F32)
    launch_kernel(gated_residual_kernel<float>, dim3(T), dim3(threads), 0, stream, x, y, y_bias, g, ldg, gate_bias, history,
                  hist_stride, n_hist, avg, norm_w, eps, (float*)out, d, clear_y, clear_g);
  else if (out_dtype == DLGO_BF16)
    launch_kernel(gated_residual_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, x, y, y_bias, g, ldg, gate_bias,
                  history, hist_stride, n_hist, avg, norm_w, eps, (__nv_bfloat16*)out, d, clear_y, clear_g);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

DLGO_EXPORT int dlgo_scale_softcap(float* z, long long n, float scale, float cap, cudaStream_t stream) {
  if (n <= 0) return DLGO_OK;
  launch_kernel(scale_softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, z, n, scale, cap);
  return launch_status();
}
