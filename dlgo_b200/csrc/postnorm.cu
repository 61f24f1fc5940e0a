// The hand-over of a layer that norms AFTER the residual sum:
//
//   u = skip * x + ls * y          (skip a constant, ls one number per channel or absent, y a sublayer's result)
//   x <- u / sqrt(mean(u^2) + eps) * w
//
// x [T, d] is the fp32 residual stream, rewritten in place; y [T, d] is fp32 and, with `clear_y`, left zero
// for the next sublayer to add into; the new x is also written in the run's type (`act`) for the
// contractions that read it next.  Sum, statistics and norm are fp32.  With y == nullptr and w == nullptr
// the kernel only makes the copy in the run's type (the first layer's input).
//
// Rows of a multiple of four numbers up to 4,096: a block per row that keeps the row in registers between the
// two passes, 16-byte accesses.  Other rows: a block per row, or a warp per row where rows are many and short.
// Either way a row's result depends on nothing else in the launch.
#include "common.cuh"

namespace dlgo {

template <typename T, bool WARP_ROW>
__global__ void __launch_bounds__(256)
scaled_add_rmsnorm_kernel(float* x, float* y, const float* __restrict__ ls,
                          const float* __restrict__ w, T* act, int rows, int d, float skip, float eps,
                          int clear_y) {
  __shared__ float red[32];
  pdl_launch_dependents();
  const int row = WARP_ROW ? blockIdx.x * 8 + (threadIdx.x >> 5) : blockIdx.x;
  const int tid = WARP_ROW ? (threadIdx.x & 31) : threadIdx.x;
  const int step = WARP_ROW ? 32 : blockDim.x;
  pdl_wait();
  if (WARP_ROW && row >= rows) return;
  float* xr = x + (size_t)row * d;
  float* yr = y == nullptr ? nullptr : y + (size_t)row * d;
  T* ar = act == nullptr ? nullptr : act + (size_t)row * d;
  if (w == nullptr) {            // copy only
    for (int i = tid; i < d; i += step) ar[i] = from_float<T>(xr[i]);
    return;
  }
  float ss = 0.f;
  for (int i = tid; i < d; i += step) {
    float u = skip * xr[i];
    if (yr != nullptr) {
      const float v = yr[i];
      u += (ls != nullptr ? ls[i] : 1.0f) * v;
    }
    xr[i] = u;                   // each thread reads back only what it wrote itself
    ss += u * u;
  }
  ss = WARP_ROW ? warp_sum(ss) : block_sum(ss, red);
  const float r = 1.0f / sqrtf(ss / (float)d + eps);
  for (int i = tid; i < d; i += step) {
    const float v = xr[i] * r * w[i];
    xr[i] = v;
    if (ar != nullptr) ar[i] = from_float<T>(v);
    if (yr != nullptr && clear_y) yr[i] = 0.f;
  }
}

// The same with the row held in registers between the two passes: a block per row, 16-byte accesses, for rows of a
// multiple of four numbers up to THREADS * 16.
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 o;
  o.x = *reinterpret_cast<unsigned*>(&a);
  o.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = o;
}

template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
scaled_add_rmsnorm_vec_kernel(float* x, float* y, const float* __restrict__ ls,
                              const float* __restrict__ w, T* act, int d, float skip, float eps,
                              int clear_y) {
  constexpr int NV = 4;
  __shared__ float red[32];
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  float4 lsv[NV], wv[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {       // weights: nothing of the step writes them
    const int i = (v * THREADS + tid) * 4;
    if (i < d) {
      lsv[v] = ls != nullptr ? *reinterpret_cast<const float4*>(ls + i) : make_float4(1.f, 1.f, 1.f, 1.f);
      wv[v] = *reinterpret_cast<const float4*>(w + i);
    }
  }
  pdl_wait();
  float* xr = x + (size_t)blockIdx.x * d;
  float* yr = y == nullptr ? nullptr : y + (size_t)blockIdx.x * d;
  float4 u[NV];
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int i = (v * THREADS + tid) * 4;
    if (i < d) {
      float4 a = *reinterpret_cast<const float4*>(xr + i);
      a.x *= skip; a.y *= skip; a.z *= skip; a.w *= skip;
      if (yr != nullptr) {
        const float4 b = *reinterpret_cast<const float4*>(yr + i);
        a.x += lsv[v].x * b.x; a.y += lsv[v].y * b.y; a.z += lsv[v].z * b.z; a.w += lsv[v].w * b.w;
      }
      u[v] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  ss = block_sum(ss, red);
  const float r = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int i = (v * THREADS + tid) * 4;
    if (i < d) {
      float4 o;
      o.x = u[v].x * r * wv[v].x; o.y = u[v].y * r * wv[v].y; o.z = u[v].z * r * wv[v].z; o.w = u[v].w * r * wv[v].w;
      *reinterpret_cast<float4*>(xr + i) = o;
      if (act != nullptr) store4<T>(act + (size_t)blockIdx.x * d + i, o);
      // (cleared here, with the other stores: a store to y right behind its load held every load of the row up,
      // 74 against 18 us for 2,048 rows of 2,048)
      if (yr != nullptr && clear_y) *reinterpret_cast<float4*>(yr + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

template <typename T>
int launch_scaled_add_rmsnorm(float* x, float* y, const float* ls, const float* w, void* act, int rows, int d,
                              float skip, float eps, int clear_y, cudaStream_t stream) {
  const bool aligned = ((uintptr_t)x % 16) == 0 && (y == nullptr || ((uintptr_t)y % 16) == 0) &&
                       (ls == nullptr || ((uintptr_t)ls % 16) == 0) && ((uintptr_t)w % 16) == 0 &&
                       (act == nullptr || ((uintptr_t)act % 16) == 0);
  if (w != nullptr && d % 4 == 0 && d <= 4096 && aligned) {
    if (d <= 1024)
      launch_kernel(scaled_add_rmsnorm_vec_kernel<T, 64>, dim3(rows), dim3(64), 0, stream, x, y, ls, w, (T*)act, d, skip,
                    eps, clear_y);
    else if (d <= 2048)
      launch_kernel(scaled_add_rmsnorm_vec_kernel<T, 128>, dim3(rows), dim3(128), 0, stream, x, y, ls, w, (T*)act, d,
                    skip, eps, clear_y);
    else
      launch_kernel(scaled_add_rmsnorm_vec_kernel<T, 256>, dim3(rows), dim3(256), 0, stream, x, y, ls, w, (T*)act, d,
                    skip, eps, clear_y);
    return launch_status();
  }
  if (rows > 64 && d <= 1024) {
    launch_kernel(scaled_add_rmsnorm_kernel<T, true>, dim3((rows + 7) / 8), dim3(256), 0, stream, x, y, ls, w, (T*)act,
                  rows, d, skip, eps, clear_y);
  } else {
    const int threads = d >= 2048 ? 256 : (d >= 512 ? 128 : 64);
    launch_kernel(scaled_add_rmsnorm_kernel<T, false>, dim3(rows), dim3(threads), 0, stream, x, y, ls, w, (T*)act, rows,
                  d, skip, eps, clear_y);
  }
  return launch_status();
}

}  // namespace dlgo

DLGO_EXPORT int dlgo_scaled_add_rmsnorm(float* x, float* y, const float* ls, const float* w, void* act, int dtype,
                                        int rows, int d, float skip, float eps, int clear_y, cudaStream_t stream) {
  if (rows <= 0) return DLGO_OK;
  if (d <= 0) return DLGO_ERR_SIZE;
  if (w == nullptr && (act == nullptr || y != nullptr)) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32)
    return dlgo::launch_scaled_add_rmsnorm<float>(x, y, ls, w, act, rows, d, skip, eps, clear_y, stream);
  if (dtype == DLGO_BF16)
    return dlgo::launch_scaled_add_rmsnorm<__nv_bfloat16>(x, y, ls, w, act, rows, d, skip, eps, clear_y, stream);
  return DLGO_ERR_DTYPE;
}
