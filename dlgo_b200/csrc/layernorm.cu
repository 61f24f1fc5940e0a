// Layer norm with a weight and no bias, and the hand-over of a layer that norms a sublayer's RESULT before it
// joins the residual stream:
//
//   LN(u) = (u - mean(u)) / sqrt(mean((u - mean(u))^2) + eps) * w        (the variance is the mean of the squared
//                                                                          deviations: two passes over the row)
//   RMS(u) = u / sqrt(mean(u^2) + eps) * w
//
// layernorm_rows:  out[r] = N(x[rows[r]])  for fp32 rows x [T, d], into the run's type or fp32 (out may be x itself:
//                  the norm of the embedding rewrites the stream in place).
// add_normed:      x <- x + N(y)  on the fp32 residual stream x [T, d]; y [T, d] is the sublayer's fp32 result and,
//                  with `clear_y`, is left zero for the next sublayer to add into; the new x is also written in the
//                  run's type (`act`) for the contractions that read it next.
//
// N is the layer norm (kind 0) or the RMS norm (kind 1).  Statistics, norm and sum are fp32.  Rows of a multiple of
// four numbers up to 4,096 stay in registers between the passes (a block per row, 16-byte accesses); other rows
// are read again from memory.  A row's result depends on nothing else in the launch.
#include "common.cuh"

namespace dlgo {

enum { NORMED_LAYER = 0, NORMED_RMS = 1 };

template <typename T> __device__ __forceinline__ void ln_store4(T* p, float4 v);
template <> __device__ __forceinline__ void ln_store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void ln_store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 o;
  o.x = *reinterpret_cast<unsigned*>(&a);
  o.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = o;
}

// (shift, scale) of a row held as NV float4 per thread: LN: (mean, 1 / sqrt(var + eps)); RMS: (0, 1 / sqrt(ms + eps))
template <int NV, int THREADS>
__device__ __forceinline__ void row_stats(const float4 (&u)[NV], int d, int tid, int kind, float eps, float* red,
                                          float& shift, float& scale) {
  float s = 0.f;
  shift = 0.f;
  if (kind == NORMED_LAYER) {
#pragma unroll
    for (int v = 0; v < NV; ++v)
      if ((v * THREADS + tid) * 4 < d) s += (u[v].x + u[v].y) + (u[v].z + u[v].w);
    shift = block_sum(s, red) / (float)d;
    s = 0.f;
  }
#pragma unroll
  for (int v = 0; v < NV; ++v)
    if ((v * THREADS + tid) * 4 < d) {
      const float a = u[v].x - shift, b = u[v].y - shift, c = u[v].z - shift, e = u[v].w - shift;
      s += (a * a + b * b) + (c * c + e * e);
    }
  scale = 1.0f / sqrtf(block_sum(s, red) / (float)d + eps);
}

template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
add_normed_vec_kernel(float* x, float* y, const float* __restrict__ w, T* act,
                      int d, int kind, float eps, int clear_y) {
  constexpr int NV = 4;
  __shared__ float red[32];
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  float4 wv[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {       // weights: nothing of the step writes them
    const int i = (v * THREADS + tid) * 4;
    if (i < d) wv[v] = *reinterpret_cast<const float4*>(w + i);
  }
  pdl_wait();
  float* xr = x + (size_t)blockIdx.x * d;
  float* yr = y + (size_t)blockIdx.x * d;
  float4 u[NV], xv[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int i = (v * THREADS + tid) * 4;
    if (i < d) {
      u[v] = *reinterpret_cast<const float4*>(yr + i);
      xv[v] = *reinterpret_cast<const float4*>(xr + i);
    }
  }
  float shift, scale;
  row_stats<NV, THREADS>(u, d, tid, kind, eps, red, shift, scale);
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int i = (v * THREADS + tid) * 4;
    if (i < d) {
      float4 o;
      o.x = xv[v].x + (u[v].x - shift) * scale * wv[v].x;
      o.y = xv[v].y + (u[v].y - shift) * scale * wv[v].y;
      o.z = xv[v].z + (u[v].z - shift) * scale * wv[v].z;
      o.w = xv[v].w + (u[v].w - shift) * scale * wv[v].w;
      *reinterpret_cast<float4*>(xr + i) = o;
      if (act != nullptr) ln_store4<T>(act + (size_t)blockIdx.x * d + i, o);
      if (clear_y) *reinterpret_cast<float4*>(yr + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

// any row length: the row is read again for every pass
template <typename T>
__global__ void __launch_bounds__(256)
add_normed_kernel(float* x, float* y, const float* __restrict__ w, T* act, int d,
                  int kind, float eps, int clear_y) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  float* xr = x + (size_t)blockIdx.x * d;
  float* yr = y + (size_t)blockIdx.x * d;
  float shift = 0.f, s = 0.f;
  if (kind == NORMED_LAYER) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) s += yr[i];
    shift = block_sum(s, red) / (float)d;
    s = 0.f;
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float a = yr[i] - shift;
    s += a * a;
  }
  const float scale = 1.0f / sqrtf(block_sum(s, red) / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float o = xr[i] + (yr[i] - shift) * scale * w[i];
    xr[i] = o;
    if (act != nullptr) act[(size_t)blockIdx.x * d + i] = from_float<T>(o);
    if (clear_y) yr[i] = 0.f;
  }
}

// out[r] = N(x[rows[r]]) (rows null: row r); out may alias x when rows is null and T is float
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
layernorm_rows_vec_kernel(const float* x, const float* __restrict__ w, T* out, const int* __restrict__ rows, int d,
                          int kind, float eps) {
  constexpr int NV = 4;
  __shared__ float red[32];
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  float4 wv[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int i = (v * THREADS + tid) * 4;
    if (i < d) wv[v] = *reinterpret_cast<const float4*>(w + i);
  }
  const int row = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;      // (the step's own input)
  pdl_wait();
  const float* xr = x + (size_t)row * d;
  float4 u[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int i = (v * THREADS + tid) * 4;
    if (i < d) u[v] = *reinterpret_cast<const float4*>(xr + i);
  }
  float shift, scale;
  row_stats<NV, THREADS>(u, d, tid, kind, eps, red, shift, scale);
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int i = (v * THREADS + tid) * 4;
    if (i < d) {
      float4 o;
      o.x = (u[v].x - shift) * scale * wv[v].x;
      o.y = (u[v].y - shift) * scale * wv[v].y;
      o.z = (u[v].z - shift) * scale * wv[v].z;
      o.w = (u[v].w - shift) * scale * wv[v].w;
      ln_store4<T>(out + (size_t)blockIdx.x * d + i, o);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
layernorm_rows_kernel(const float* x, const float* __restrict__ w, T* out, const int* __restrict__ rows, int d, int kind,
                      float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  const int row = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
  pdl_wait();
  const float* xr = x + (size_t)row * d;
  float shift = 0.f, s = 0.f;
  if (kind == NORMED_LAYER) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) s += xr[i];
    shift = block_sum(s, red) / (float)d;
    s = 0.f;
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float a = xr[i] - shift;
    s += a * a;
  }
  const float scale = 1.0f / sqrtf(block_sum(s, red) / (float)d + eps);   // (a barrier: every read of the row is done)
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = xr[i];
    out[(size_t)blockIdx.x * d + i] = from_float<T>((v - shift) * scale * w[i]);
  }
}

template <typename T>
int launch_add_normed(float* x, float* y, const float* w, void* act, int rows, int d, int kind, float eps, int clear_y,
                      cudaStream_t stream) {
  const bool aligned = ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)w % 16) == 0 &&
                       (act == nullptr || ((uintptr_t)act % 16) == 0);
  if (d % 4 == 0 && d <= 4096 && aligned) {
    if (d <= 1024)
      launch_kernel(add_normed_vec_kernel<T, 64>, dim3(rows), dim3(64), 0, stream, x, y, w, (T*)act, d, kind, eps, clear_y);
    else if (d <= 2048)
      launch_kernel(add_normed_vec_kernel<T, 128>, dim3(rows), dim3(128), 0, stream, x, y, w, (T*)act, d, kind, eps, clear_y);
    else
      launch_kernel(add_normed_vec_kernel<T, 256>, dim3(rows), dim3(256), 0, stream, x, y, w, (T*)act, d, kind, eps, clear_y);
    return launch_status();
  }
  const int threads = d >= 2048 ? 256 : (d >= 512 ? 128 : 64);
  launch_kernel(add_normed_kernel<T>, dim3(rows), dim3(threads), 0, stream, x, y, w, (T*)act, d, kind, eps, clear_y);
  return launch_status();
}

template <typename T>
int launch_layernorm_rows(const float* x, const float* w, void* out, const int* rows, int R, int d, int kind, float eps,
                          cudaStream_t stream) {
  const bool aligned = ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 16) == 0;
  if (d % 4 == 0 && d <= 4096 && aligned) {
    if (d <= 1024)
      launch_kernel(layernorm_rows_vec_kernel<T, 64>, dim3(R), dim3(64), 0, stream, x, w, (T*)out, rows, d, kind, eps);
    else if (d <= 2048)
      launch_kernel(layernorm_rows_vec_kernel<T, 128>, dim3(R), dim3(128), 0, stream, x, w, (T*)out, rows, d, kind, eps);
    else
      launch_kernel(layernorm_rows_vec_kernel<T, 256>, dim3(R), dim3(256), 0, stream, x, w, (T*)out, rows, d, kind, eps);
    return launch_status();
  }
  const int threads = d >= 2048 ? 256 : (d >= 512 ? 128 : 64);
  launch_kernel(layernorm_rows_kernel<T>, dim3(R), dim3(threads), 0, stream, x, w, (T*)out, rows, d, kind, eps);
  return launch_status();
}

}  // namespace dlgo

// x [rows, d] fp32 (in place), y [rows, d] fp32, w [d] fp32, act [rows, d] in `dtype` or null
DLGO_EXPORT int dlgo_add_normed(float* x, float* y, const float* w, void* act, int dtype, int rows, int d, int kind,
                                float eps, int clear_y, cudaStream_t stream) {
  if (rows <= 0) return DLGO_OK;
  if (d <= 0 || x == nullptr || y == nullptr || w == nullptr) return DLGO_ERR_SIZE;
  if (kind != dlgo::NORMED_LAYER && kind != dlgo::NORMED_RMS) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32) return dlgo::launch_add_normed<float>(x, y, w, act, rows, d, kind, eps, clear_y, stream);
  if (dtype == DLGO_BF16) return dlgo::launch_add_normed<__nv_bfloat16>(x, y, w, act, rows, d, kind, eps, clear_y, stream);
  return DLGO_ERR_DTYPE;
}

// out [R, d] in `dtype`: the norm of rows `rows` (int32 [R]; null: rows 0..R-1, and out may then be x itself in fp32)
DLGO_EXPORT int dlgo_layernorm_rows(const float* x, const float* w, void* out, int dtype, const int* rows, int R, int d,
                                    int kind, float eps, cudaStream_t stream) {
  if (R <= 0) return DLGO_OK;
  if (d <= 0 || x == nullptr || w == nullptr || out == nullptr) return DLGO_ERR_SIZE;
  if (kind != dlgo::NORMED_LAYER && kind != dlgo::NORMED_RMS) return DLGO_ERR_SIZE;
  if (out == (const void*)x && (rows != nullptr || dtype != DLGO_F32)) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32) return dlgo::launch_layernorm_rows<float>(x, w, out, rows, R, d, kind, eps, stream);
  if (dtype == DLGO_BF16) return dlgo::launch_layernorm_rows<__nv_bfloat16>(x, w, out, rows, R, d, kind, eps, stream);
  return DLGO_ERR_DTYPE;
}
