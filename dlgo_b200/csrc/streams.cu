// Several residual streams ("hyper-connections"), the Dynamic-Tanh norm, and the small row kernels of
// the parts that live on them.
//
//   streams  X[t, r, :] for r < s, fp32.  A sublayer reads u = sum_r a[r] X[t, r, :], runs on norm(u), and its
//            result y goes back into every stream at once, from the old values:
//            X'[t, q, :] = sum_r M[r, q] X[t, r, :] + b[q] * y[t, :]            (M indexed [from, to])
//   norms    Dynamic Tanh: tanh(alpha * u) * w + beta (no statistics); RMS: u / sqrt(mean(u^2) + eps) * w
//   bias_act act(z + bias): none, relu(z)^2, silu, tanh-form gelu, tanh
//   gated    rms(o) * w * gate(g) * c, the mean over the whole row or over each group of neighbours (a head);
//            gate is sigmoid or silu, w may be absent
//
// One launch does a whole hand-over between two sublayers: the write of sublayer k's result, the read for
// sublayer k+1 and its norm.  Everything is computed in fp32; TO is the type handed to the next contraction.
#include "common.cuh"

namespace dlgo {

constexpr int MAX_STREAMS = 8;
enum { NORM_NONE = 0, NORM_RMS = 1, NORM_DYT = 2 };
enum { ACT_NONE = 0, ACT_RELU2 = 1, ACT_SILU = 2, ACT_GELU_TANH = 3, ACT_TANH = 4 };
enum { GATE_SIGMOID = 0, GATE_SILU = 1 };

struct StreamsStep {
  float* X;             // [T, s, d]
  int s, d;
  // write part (y == nullptr: none)
  float* y;             // [T, d] the sublayer's result; left zero when clear_y
  const float* y_bias;  // [d] added to y first, or null
  const float* mix;     // [s, s] (from, to)
  const float* wout;    // [s]
  int clear_y;
  // read part (norm_kind == NORM_NONE and out == nullptr: none)
  const float* coeff;   // [s], or null for the plain sum of the streams
  int norm_kind;
  const float* nw;      // [d]
  const float* nb;      // [d] (Dynamic Tanh) or null
  const float* nalpha;  // [1] (Dynamic Tanh)
  float eps;
  void* out;            // [R, d]
  const int* rows;      // [R] rows of X to read (read part only), or null
};

template <typename TO> __device__ __forceinline__ void store4(TO* o, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* o, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* o, float a, float b, float c, float d) {
  __nv_bfloat162 h[2] = {__floats2bfloat162_rn(a, b), __floats2bfloat162_rn(c, d)};
  *reinterpret_cast<uint2*>(o) = *reinterpret_cast<uint2*>(h);
}

template <typename TO>
__global__ void __launch_bounds__(256) streams_step_kernel(StreamsStep p) {
  pdl_launch_dependents();
  __shared__ float s_mix[MAX_STREAMS * MAX_STREAMS], s_wout[MAX_STREAMS], s_coeff[MAX_STREAMS];
  __shared__ float scratch[32];
  __shared__ float scale_s;
  const int s = p.s, d = p.d;
  // coefficients are weights: fetched before the wait for the predecessor
  if (threadIdx.x < s * s && p.y) s_mix[threadIdx.x] = p.mix[threadIdx.x];
  if (threadIdx.x < s) {
    if (p.y) s_wout[threadIdx.x] = p.wout[threadIdx.x];
    s_coeff[threadIdx.x] = p.coeff ? p.coeff[threadIdx.x] : 1.0f;
  }
  const float alpha = (p.norm_kind == NORM_DYT) ? p.nalpha[0] : 0.f;
  const int r = blockIdx.x;
  const int row = p.rows ? p.rows[r] : r;
  __syncthreads();
  pdl_wait();
  float* xr = p.X + (size_t)row * s * d;
  float* yr = p.y ? p.y + (size_t)row * d : nullptr;
  TO* o = p.out ? reinterpret_cast<TO*>(p.out) + (size_t)r * d : nullptr;
  float ss = 0.f;
  // four columns per thread and trip (16-byte accesses) where the row length allows, else one
  const int W = (d & 3) == 0 ? 4 : 1;
  for (int i0 = threadIdx.x * W; i0 < d; i0 += blockDim.x * W) {
    float x[MAX_STREAMS][4];
#pragma unroll
    for (int a = 0; a < MAX_STREAMS; ++a) {
      if (a < s) {
        if (W == 4) {
          const float4 v = *reinterpret_cast<const float4*>(xr + (size_t)a * d + i0);
          x[a][0] = v.x; x[a][1] = v.y; x[a][2] = v.z; x[a][3] = v.w;
        } else {
          x[a][0] = xr[(size_t)a * d + i0];
          x[a][1] = x[a][2] = x[a][3] = 0.f;
        }
      }
    }
    if (yr) {
      float yv[4] = {0.f, 0.f, 0.f, 0.f};
      if (W == 4) {
        const float4 v = *reinterpret_cast<const float4*>(yr + i0);
        yv[0] = v.x; yv[1] = v.y; yv[2] = v.z; yv[3] = v.w;
        if (p.y_bias) {
          const float4 b = *reinterpret_cast<const float4*>(p.y_bias + i0);
          yv[0] += b.x; yv[1] += b.y; yv[2] += b.z; yv[3] += b.w;
        }
        if (p.clear_y) *reinterpret_cast<float4*>(yr + i0) = make_float4(0.f, 0.f, 0.f, 0.f);
      } else {
        yv[0] = yr[i0] + (p.y_bias ? p.y_bias[i0] : 0.f);
        if (p.clear_y) yr[i0] = 0.f;
      }
      float nx[MAX_STREAMS][4];
#pragma unroll
      for (int q = 0; q < MAX_STREAMS; ++q) {
        if (q < s) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float acc = 0.f;
#pragma unroll
            for (int a = 0; a < MAX_STREAMS; ++a)
              if (a < s) acc = fmaf(s_mix[a * s + q], x[a][c], acc);
            nx[q][c] = fmaf(s_wout[q], yv[c], acc);
          }
          if (W == 4)
            *reinterpret_cast<float4*>(xr + (size_t)q * d + i0) = make_float4(nx[q][0], nx[q][1], nx[q][2], nx[q][3]);
          else
            xr[(size_t)q * d + i0] = nx[q][0];
        }
      }
#pragma unroll
      for (int q = 0; q < MAX_STREAMS; ++q)
        if (q < s) {
#pragma unroll
          for (int c = 0; c < 4; ++c) x[q][c] = nx[q][c];
        }
    }
    if (o) {
      float u[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        u[c] = 0.f;
#pragma unroll
        for (int a = 0; a < MAX_STREAMS; ++a)
          if (a < s) u[c] = fmaf(s_coeff[a], x[a][c], u[c]);
      }
      if (p.norm_kind == NORM_RMS) {
        for (int c = 0; c < W; ++c) ss = fmaf(u[c], u[c], ss);
      } else {
        float r4[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int i = i0 + (c < W ? c : 0);
          r4[c] = p.norm_kind == NORM_DYT ? fmaf(tanhf(alpha * u[c]), p.nw[i], p.nb ? p.nb[i] : 0.f) : u[c];
        }
        if (W == 4) store4<TO>(o + i0, r4[0], r4[1], r4[2], r4[3]);
        else o[i0] = from_float<TO>(r4[0]);
      }
    }
  }
  if (o && p.norm_kind == NORM_RMS) {
    ss = block_sum(ss, scratch);
    if (threadIdx.x == 0) scale_s = 1.0f / sqrtf(ss / (float)d + p.eps);
    __syncthreads();
    const float sc = scale_s;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {      // each thread re-reads what it wrote itself
      float u = 0.f;
      for (int a = 0; a < s; ++a) u = fmaf(s_coeff[a], xr[(size_t)a * d + i], u);
      o[i] = from_float<TO>(u * sc * p.nw[i]);
    }
  }
}

__device__ __forceinline__ float activate(float z, int act) {
  switch (act) {
    case ACT_RELU2: { const float r = fmaxf(z, 0.f); return r * r; }
    case ACT_SILU: return z / (1.0f + expf(-z));
    case ACT_GELU_TANH: return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    case ACT_TANH: return tanhf(z);
    default: return z;
  }
}

// out[t, i] = act(z[t, i] + bias[i]); z fp32 with row stride ldz; out may be z itself (fp32, same stride)
template <typename TO>
__global__ void bias_act_kernel(const float* z, int ldz, const float* __restrict__ bias, TO* out, int ldo, int T, int n,
                                int act) {
  pdl_launch_dependents();
  pdl_wait();
  if ((n & 3) == 0 && (ldz & 3) == 0 && (ldo & 3) == 0 && ((uintptr_t)z & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
      (bias == nullptr || ((uintptr_t)bias & 15) == 0)) {
    const int n4 = n >> 2;
    const size_t total4 = (size_t)T * n4;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total4; e += (size_t)gridDim.x * blockDim.x) {
      const int t = (int)(e / n4), i = (int)(e % n4) * 4;
      float4 v = *reinterpret_cast<const float4*>(z + (size_t)t * ldz + i);
      if (bias) {
        const float4 b = __ldg(reinterpret_cast<const float4*>(bias + i));
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
      }
      store4<TO>(out + (size_t)t * ldo + i, activate(v.x, act), activate(v.y, act), activate(v.z, act), activate(v.w, act));
    }
    return;
  }
  const size_t total = (size_t)T * n;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(e / n), i = (int)(e % n);
    const float v = z[(size_t)t * ldz + i] + (bias ? bias[i] : 0.f);
    out[(size_t)t * ldo + i] = from_float<TO>(activate(v, act));
  }
}

__device__ __forceinline__ float gate_of(float g, int gate_act) {
  const float sg = 1.0f / (1.0f + expf(-g));
  return gate_act == GATE_SILU ? g * sg : sg;
}

// out[t, :] = o[t, :] / sqrt(mean(o[t, :]^2) + eps) * w * gate(g[t, :]) * c;  o, g fp32 with row strides; w may be null
template <typename TO>
__global__ void gated_rmsnorm_kernel(const float* o, int ldo, const float* g, int ldg,
                                     const float* __restrict__ w, TO* out, int n, float eps, int gate_act,
                                     float c) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  __shared__ float scale_s;
  pdl_wait();
  const int t = blockIdx.x;
  const float* orow = o + (size_t)t * ldo;
  const float* grow = g + (size_t)t * ldg;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(orow[i], orow[i], ss);
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) scale_s = 1.0f / sqrtf(ss / (float)n + eps);
  __syncthreads();
  const float sc = scale_s * c;
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    out[(size_t)t * n + i] = from_float<TO>(orow[i] * sc * (w != nullptr ? w[i] : 1.0f) * gate_of(grow[i], gate_act));
}

// The same with the mean taken over each group of `group` neighbours (a head) on its own: a warp per (token, group).
constexpr int GG_WARPS = 4;
template <typename TO>
__global__ void __launch_bounds__(GG_WARPS * 32)
gated_groupnorm_kernel(const float* o, int ldo, const float* g, int ldg,
                       const float* __restrict__ w, TO* out, int T, int n, int group, float eps,
                       int gate_act, float c) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int groups = n / group;
  const long long item = (long long)blockIdx.x * GG_WARPS + warp;
  pdl_wait();
  if (item >= (long long)T * groups) return;
  const int t = (int)(item / groups), gi = (int)(item - (long long)t * groups);
  const float* orow = o + (size_t)t * ldo + (size_t)gi * group;
  const float* grow = g + (size_t)t * ldg + (size_t)gi * group;
  float ss = 0.f;
  for (int i = lane; i < group; i += 32) ss = fmaf(orow[i], orow[i], ss);
  ss = warp_sum(ss);
  const float sc = c / sqrtf(ss / (float)group + eps);
  for (int i = lane; i < group; i += 32)
    out[(size_t)t * n + (size_t)gi * group + i] =
        from_float<TO>(orow[i] * sc * (w != nullptr ? w[(size_t)gi * group + i] : 1.0f) * gate_of(grow[i], gate_act));
}

}  // namespace dlgo

using namespace dlgo;

DLGO_EXPORT int dlgo_streams_step(float* X, int T, int s, int d, float* y, const float* y_bias, const float* mix,
                                  const float* wout, int clear_y, const float* coeff, int norm_kind, const float* nw,
                                  const float* nb, const float* nalpha, float eps, void* out, int out_dtype,
                                  const int* rows, int R, cudaStream_t stream) {
  if (s < 1 || s > MAX_STREAMS || d <= 0) return DLGO_ERR_SIZE;
  if (y && rows) return DLGO_ERR_SIZE;      // the write part runs on every row
  const int n_rows = y ? T : R;
  if (n_rows <= 0) return DLGO_OK;
  if (out && out_dtype != DLGO_F32 && out_dtype != DLGO_BF16) return DLGO_ERR_DTYPE;
  if (out && norm_kind != NORM_NONE && !nw) return DLGO_ERR_SIZE;
  StreamsStep p{X, s, d, y, y_bias, mix, wout, clear_y, coeff, norm_kind, nw, nb, nalpha, eps, out, rows};
  const int threads = d >= 1024 ? 256 : 128;      // (four columns per thread and trip)
  if (out && out_dtype == DLGO_BF16)
    launch_kernel(streams_step_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, p);
  else
    launch_kernel(streams_step_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, p);
  return launch_status();
}

DLGO_EXPORT int dlgo_bias_act(const float* z, int ldz, const float* bias, void* out, int out_dtype, int ldo, int T,
                              int n, int act, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return DLGO_OK;
  if (act < ACT_NONE || act > ACT_TANH) return DLGO_ERR_SIZE;
  const size_t total = ((size_t)T * n + 3) / 4;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (out_dtype == DLGO_F32)
    launch_kernel(bias_act_kernel<float>, dim3(blocks), dim3(threads), 0, stream, z, ldz, bias, (float*)out, ldo, T, n, act);
  else if (out_dtype == DLGO_BF16)
    launch_kernel(bias_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, z, ldz, bias,
                  (__nv_bfloat16*)out, ldo, T, n, act);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

// group: numbers per group whose mean square is taken together (n: the whole row); gate_act: GATE_*; c: a constant factor
DLGO_EXPORT int dlgo_gated_rmsnorm(const float* o, int ldo, const float* g, int ldg, const float* w, void* out,
                                   int out_dtype, int T, int n, float eps, int group, int gate_act, float c,
                                   cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (n <= 0 || group <= 0 || n % group || (gate_act != GATE_SIGMOID && gate_act != GATE_SILU)) return DLGO_ERR_SIZE;
  if (out_dtype != DLGO_F32 && out_dtype != DLGO_BF16) return DLGO_ERR_DTYPE;
  if (group < n) {
    const long long items = (long long)T * (n / group);
    const long long blocks = (items + GG_WARPS - 1) / GG_WARPS;
    if (blocks > 0x7fffffffLL) return DLGO_ERR_SIZE;
    if (out_dtype == DLGO_F32)
      launch_kernel(gated_groupnorm_kernel<float>, dim3((unsigned)blocks), dim3(GG_WARPS * 32), 0, stream, o, ldo, g, ldg,
                    w, (float*)out, T, n, group, eps, gate_act, c);
    else
      launch_kernel(gated_groupnorm_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(GG_WARPS * 32), 0, stream, o, ldo,
                    g, ldg, w, (__nv_bfloat16*)out, T, n, group, eps, gate_act, c);
    return launch_status();
  }
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
  if (out_dtype == DLGO_F32)
    launch_kernel(gated_rmsnorm_kernel<float>, dim3(T), dim3(threads), 0, stream, o, ldo, g, ldg, w, (float*)out, n, eps,
                  gate_act, c);
  else
    launch_kernel(gated_rmsnorm_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, o, ldo, g, ldg, w,
                  (__nv_bfloat16*)out, n, eps, gate_act, c);
  return launch_status();
}
