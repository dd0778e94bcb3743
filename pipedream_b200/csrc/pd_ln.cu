// LayerNorm over the last dimension and GELU, forward and backward, for the transformer stage modules of the
// 2BW configuration (the reference ships no GPT stage files; torch.nn.LayerNorm / torch.nn.GELU are what such
// stages are built from).  Both are HBM-bound: one warp per row for LayerNorm (the row stays in registers
// between the statistics and the normalisation), 16-byte accesses for bf16; parameter gradients are reduced in
// two deterministic levels (per-block partial column sums, then one block per 32 columns).
#include "pd_common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxPerLane = 32;          // C <= 1024

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// y = (x - mean) * rstd * gamma + beta, one warp per row; mean / rstd saved in fp32.
template <typename T>
__global__ void __launch_bounds__(kThreads)
layernorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, int64_t rows, int C,
                     float eps, T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int per = (C + 31) / 32;
  for (int64_t r = warp0; r < rows; r += (int64_t)gridDim.x * kWarps) {
    const T* xr = x + r * C;
    float v[kMaxPerLane];
    float s = 0.f;
#pragma unroll 8
    for (int k = 0; k < per; ++k) {
      const int c = lane + k * 32;
      v[k] = c < C ? pd_to_float(xr[c]) : 0.f;
      s += v[k];
    }
    const float m = warp_sum(s) / (float)C;
    float q = 0.f;
#pragma unroll 8
    for (int k = 0; k < per; ++k) {
      const int c = lane + k * 32;
      const float d = c < C ? v[k] - m : 0.f;
      q += d * d;
    }
    const float rs = rsqrtf(warp_sum(q) / (float)C + eps);
    T* yr = y + r * C;
#pragma unroll 8
    for (int k = 0; k < per; ++k) {
      const int c = lane + k * 32;
      if (c < C) yr[c] = pd_from_float<T>((v[k] - m) * rs * pd_to_float(gamma[c]) + pd_to_float(beta[c]));
    }
    if (lane == 0) { mean[r] = m; rstd[r] = rs; }
  }
}

// dx = rstd * (g - mean_c(g) - xhat * mean_c(g * xhat)), g = dy * gamma; one warp per row.
// Each block also accumulates the column sums of dy*xhat and dy over its rows: partial[block][2][C].
template <typename T>
__global__ void __launch_bounds__(kThreads)
layernorm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ gamma,
                     const float* __restrict__ mean, const float* __restrict__ rstd, int64_t rows, int C,
                     T* __restrict__ dx, float* __restrict__ partial) {
  extern __shared__ float sh[];            // [2][C] block accumulators
  for (int i = threadIdx.x; i < 2 * C; i += kThreads) sh[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int per = (C + 31) / 32;
  float ag[kMaxPerLane], ab[kMaxPerLane];              // this lane's column sums over the warp's rows
#pragma unroll 8
  for (int k = 0; k < per; ++k) ag[k] = ab[k] = 0.f;
  for (int64_t r = warp0; r < rows; r += (int64_t)gridDim.x * kWarps) {
    const T* xr = x + r * C;
    const T* gr = dy + r * C;
    const float m = mean[r], rs = rstd[r];
    float xh[kMaxPerLane], g[kMaxPerLane];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll 8
    for (int k = 0; k < per; ++k) {
      const int c = lane + k * 32;
      if (c < C) {
        const float d = pd_to_float(gr[c]);
        xh[k] = (pd_to_float(xr[c]) - m) * rs;
        g[k] = d * pd_to_float(gamma[c]);
        s1 += g[k];
        s2 += g[k] * xh[k];
        ag[k] += d * xh[k];
        ab[k] += d;
      } else {
        xh[k] = g[k] = 0.f;
      }
    }
    s1 = warp_sum(s1) / (float)C;
    s2 = warp_sum(s2) / (float)C;
    T* dr = dx + r * C;
#pragma unroll 8
    for (int k = 0; k < per; ++k) {
      const int c = lane + k * 32;
      if (c < C) dr[c] = pd_from_float<T>(rs * (g[k] - s1 - xh[k] * s2));
    }
  }
  // warps add their sums one after the other: a fixed order, so the result does not vary from run to run
  for (int w = 0; w < kWarps; ++w) {
    if ((threadIdx.x >> 5) == w) {
#pragma unroll 8
      for (int k = 0; k < per; ++k) {
        const int c = lane + k * 32;
        if (c < C) { sh[c] += ag[k]; sh[C + c] += ab[k]; }
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < 2 * C; i += kThreads) partial[(int64_t)blockIdx.x * 2 * C + i] = sh[i];
}

// ---- bf16, C = 256 * NV (NV = 1..4): a lane owns NV 16-byte vectors of the row, everything stays in registers ----
__device__ __forceinline__ void ln_unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 t = __bfloat1622float2(p[k]);
    f[2 * k] = t.x;
    f[2 * k + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 ln_pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) p[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
  return u;
}

template <int NV>
__global__ void __launch_bounds__(kThreads)
layernorm_fwd_v8_kernel(const uint4* __restrict__ x, const uint4* __restrict__ gamma, const uint4* __restrict__ beta,
                        int64_t rows, float eps, uint4* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd) {
  constexpr int C = NV * 256;
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  float gm[NV * 8], bt[NV * 8];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    ln_unpack8(gamma[lane + 32 * k], gm + 8 * k);
    ln_unpack8(beta[lane + 32 * k], bt + 8 * k);
  }
  for (int64_t r = warp0; r < rows; r += (int64_t)gridDim.x * kWarps) {
    const uint4* xr = x + r * (C / 8);
    float v[NV * 8];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) ln_unpack8(xr[lane + 32 * k], v + 8 * k);
#pragma unroll
    for (int j = 0; j < NV * 8; ++j) s += v[j];
    const float m = warp_sum(s) / (float)C;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < NV * 8; ++j) { const float d = v[j] - m; q += d * d; }
    const float rs = rsqrtf(warp_sum(q) / (float)C + eps);
    uint4* yr = y + r * (C / 8);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[8 * k + j] - m) * rs * gm[8 * k + j] + bt[8 * k + j];
      yr[lane + 32 * k] = ln_pack8(o);
    }
    if (lane == 0) { mean[r] = m; rstd[r] = rs; }
  }
}

template <int NV>
__global__ void __launch_bounds__(kThreads)
layernorm_bwd_v8_kernel(const uint4* __restrict__ x, const uint4* __restrict__ dy, const uint4* __restrict__ gamma,
                        const float* __restrict__ mean, const float* __restrict__ rstd, int64_t rows,
                        uint4* __restrict__ dx, float* __restrict__ partial) {
  constexpr int C = NV * 256;
  extern __shared__ float sh[];            // [2][C] block accumulators
  for (int i = threadIdx.x; i < 2 * C; i += kThreads) sh[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  float gm[NV * 8], ag[NV * 8], ab[NV * 8];
#pragma unroll
  for (int k = 0; k < NV; ++k) ln_unpack8(gamma[lane + 32 * k], gm + 8 * k);
#pragma unroll
  for (int j = 0; j < NV * 8; ++j) ag[j] = ab[j] = 0.f;
  for (int64_t r = warp0; r < rows; r += (int64_t)gridDim.x * kWarps) {
    const uint4* xr = x + r * (C / 8);
    const uint4* gr = dy + r * (C / 8);
    const float m = mean[r], rs = rstd[r];
    float xh[NV * 8], g[NV * 8];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      ln_unpack8(xr[lane + 32 * k], xh + 8 * k);
      ln_unpack8(gr[lane + 32 * k], g + 8 * k);
    }
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < NV * 8; ++j) {
      const float d = g[j];
      xh[j] = (xh[j] - m) * rs;
      ag[j] += d * xh[j];
      ab[j] += d;
      g[j] = d * gm[j];
      s1 += g[j];
      s2 += g[j] * xh[j];
    }
    s1 = warp_sum(s1) / (float)C;
    s2 = warp_sum(s2) / (float)C;
    uint4* dr = dx + r * (C / 8);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (g[8 * k + j] - s1 - xh[8 * k + j] * s2);
      dr[lane + 32 * k] = ln_pack8(o);
    }
  }
  // warps add their sums one after the other (fixed order); column of element j of vector k: (lane + 32k)*8 + j
  for (int w = 0; w < kWarps; ++w) {
    if ((threadIdx.x >> 5) == w) {
#pragma unroll
      for (int k = 0; k < NV; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = (lane + 32 * k) * 8 + j;
          sh[c] += ag[8 * k + j];
          sh[C + c] += ab[8 * k + j];
        }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < 2 * C; i += kThreads) partial[(int64_t)blockIdx.x * 2 * C + i] = sh[i];
}

// second level: one block (32 x 8) per 32 columns
__global__ void __launch_bounds__(256)
layernorm_param_grad_kernel(const float* __restrict__ partial, int nblocks, int C, float* __restrict__ dgamma,
                            float* __restrict__ dbeta, int accumulate) {
  __shared__ float sh[2][8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f, q = 0.f;
  if (c < C)
    for (int b = threadIdx.y; b < nblocks; b += 8) {
      s += partial[((int64_t)b * 2) * C + c];
      q += partial[((int64_t)b * 2 + 1) * C + c];
    }
  sh[0][threadIdx.y][threadIdx.x] = s;
  sh[1][threadIdx.y][threadIdx.x] = q;
  __syncthreads();
  if (threadIdx.y != 0 || c >= C) return;
  s = q = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) { s += sh[0][j][threadIdx.x]; q += sh[1][j][threadIdx.x]; }
  dgamma[c] = accumulate ? dgamma[c] + s : s;
  dbeta[c] = accumulate ? dbeta[c] + q : q;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  const float t = tanhf(u);
  const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}
__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.7071067811865476f)); }
__device__ __forceinline__ float gelu_erf_grad(float x) {
  return 0.5f * (1.f + erff(x * 0.7071067811865476f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
gelu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n, int tanh_form) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = pd_to_float(x[i]);
    y[i] = pd_from_float<T>(tanh_form ? gelu_tanh(v) : gelu_erf(v));
  }
}
template <typename T>
__global__ void __launch_bounds__(kThreads)
gelu_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dx, int64_t n, int tanh_form) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = pd_to_float(x[i]);
    dx[i] = pd_from_float<T>(pd_to_float(dy[i]) * (tanh_form ? gelu_tanh_grad(v) : gelu_erf_grad(v)));
  }
}

// bf16, 8 elements per thread
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 t = __bfloat1622float2(p[k]);
    f[2 * k] = t.x;
    f[2 * k + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) p[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
  return u;
}
__global__ void __launch_bounds__(kThreads)
gelu_fwd_bf16x8_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int64_t nvec, int tanh_form) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(x[i], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = tanh_form ? gelu_tanh(f[k]) : gelu_erf(f[k]);
    y[i] = pack8(f);
  }
}
__global__ void __launch_bounds__(kThreads)
gelu_bwd_bf16x8_kernel(const uint4* __restrict__ x, const uint4* __restrict__ dy, uint4* __restrict__ dx, int64_t nvec,
                       int tanh_form) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float f[8], g[8];
    unpack8(x[i], f);
    unpack8(dy[i], g);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = g[k] * (tanh_form ? gelu_tanh_grad(f[k]) : gelu_erf_grad(f[k]));
    dx[i] = pack8(f);
  }
}

// about four rows per warp (the per-block tail of the backward - partial sums of 2*C floats - must stay small
// next to the rows), at most two blocks per SM
int ln_blocks(int64_t rows) {
  int64_t blocks = (rows + kWarps * 4 - 1) / (kWarps * 4);
  int64_t cap = (int64_t)pd_num_sms() * 2;
  return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}
bool ln_vec(int dtype, int C, const void* a, const void* b, const void* c, const void* d) {
  return dtype == PD_BF16 && C % 256 == 0 && C <= 1024 &&
         ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)c) | ((uintptr_t)d)) & 15) == 0;
}
int flat_grid(int64_t n) {
  int64_t blocks = (n + kThreads - 1) / kThreads;
  int64_t cap = (int64_t)pd_num_sms() * 16;
  return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

}  // namespace

#define PD_LN_T(dtype, ...)                                             \
  if (dtype == PD_F32) { using T = float; __VA_ARGS__ }                 \
  else if (dtype == PD_BF16) { using T = __nv_bfloat16; __VA_ARGS__ }   \
  else { pd_set_error("bad dtype %d", dtype); return PD_ERR_INVALID; }

// fp32 scratch the backward needs for the parameter gradients.
PD_EXPORT int64_t pd_layernorm_workspace_bytes(int64_t rows, int C) {
  return (int64_t)ln_blocks(rows) * 2 * C * sizeof(float);
}

// x, y: [rows, C]; gamma, beta: [C] in `dtype`; mean, rstd: fp32 [rows] (out, saved for backward).  C <= 1024.
PD_EXPORT int pd_layernorm_fwd(int dtype, const void* x, int64_t rows, int C, const void* gamma, const void* beta, float eps,
                               void* y, float* mean, float* rstd, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x && gamma && beta && y && mean && rstd && rows > 0 && C > 0, "pd_layernorm_fwd: bad arguments");
  PD_REQUIRE(C <= 32 * kMaxPerLane, "pd_layernorm_fwd: at most %d columns", 32 * kMaxPerLane);
  cudaStream_t s = (cudaStream_t)stream;
  if (ln_vec(dtype, C, x, gamma, beta, y)) {
    const int nb = ln_blocks(rows);
#define PD_LN_FWD(NV) layernorm_fwd_v8_kernel<NV><<<nb, kThreads, 0, s>>>((const uint4*)x, (const uint4*)gamma, (const uint4*)beta, rows, eps, (uint4*)y, mean, rstd)
    switch (C / 256) { case 1: PD_LN_FWD(1); break; case 2: PD_LN_FWD(2); break; case 3: PD_LN_FWD(3); break; default: PD_LN_FWD(4); break; }
#undef PD_LN_FWD
  } else {
    PD_LN_T(dtype, layernorm_fwd_kernel<T><<<ln_blocks(rows), kThreads, 0, s>>>((const T*)x, (const T*)gamma, (const T*)beta, rows, C,
                                                                                eps, (T*)y, mean, rstd);)
  }
  PD_LAUNCH_CHECK("layernorm_fwd_kernel");
  return PD_OK;
}

// dx: [rows, C]; dgamma, dbeta: fp32 [C] (stored, or added to when accumulate != 0).
PD_EXPORT int pd_layernorm_bwd(int dtype, const void* x, const void* dy, const void* gamma, const float* mean,
                               const float* rstd, int64_t rows, int C, void* dx, float* dgamma, float* dbeta, int accumulate,
                               void* workspace, int64_t workspace_bytes, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x && dy && gamma && mean && rstd && dx && dgamma && dbeta && workspace && rows > 0 && C > 0,
             "pd_layernorm_bwd: bad arguments");
  PD_REQUIRE(C <= 32 * kMaxPerLane, "pd_layernorm_bwd: at most %d columns", 32 * kMaxPerLane);
  PD_REQUIRE(workspace_bytes >= pd_layernorm_workspace_bytes(rows, C), "pd_layernorm_bwd: workspace too small");
  cudaStream_t s = (cudaStream_t)stream;
  const int nb = ln_blocks(rows);
  const size_t smem = (size_t)2 * C * sizeof(float);
  if (ln_vec(dtype, C, x, dy, gamma, dx)) {
#define PD_LN_BWD(NV) layernorm_bwd_v8_kernel<NV><<<nb, kThreads, smem, s>>>((const uint4*)x, (const uint4*)dy, (const uint4*)gamma, mean, rstd, rows, (uint4*)dx, (float*)workspace)
    switch (C / 256) { case 1: PD_LN_BWD(1); break; case 2: PD_LN_BWD(2); break; case 3: PD_LN_BWD(3); break; default: PD_LN_BWD(4); break; }
#undef PD_LN_BWD
  } else {
    PD_LN_T(dtype, layernorm_bwd_kernel<T><<<nb, kThreads, smem, s>>>((const T*)x, (const T*)dy, (const T*)gamma, mean, rstd, rows, C,
                                                                      (T*)dx, (float*)workspace);)
  }
  PD_LAUNCH_CHECK("layernorm_bwd_kernel");
  layernorm_param_grad_kernel<<<(C + 31) / 32, dim3(32, 8), 0, s>>>((const float*)workspace, nb, C, dgamma, dbeta, accumulate);
  PD_LAUNCH_CHECK("layernorm_param_grad_kernel");
  return PD_OK;
}

// tanh_form != 0: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) (torch.nn.GELU(approximate="tanh")); else the erf form.
PD_EXPORT int pd_gelu_fwd(int dtype, const void* x, void* y, int64_t n, int tanh_form, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x && y && n >= 0, "pd_gelu_fwd: bad arguments");
  if (n == 0) return PD_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PD_BF16 && (n % 8) == 0 && ((((uintptr_t)x) | ((uintptr_t)y)) & 15) == 0) {
    gelu_fwd_bf16x8_kernel<<<flat_grid(n / 8), kThreads, 0, s>>>((const uint4*)x, (uint4*)y, n / 8, tanh_form);
  } else {
    PD_LN_T(dtype, gelu_fwd_kernel<T><<<flat_grid(n), kThreads, 0, s>>>((const T*)x, (T*)y, n, tanh_form);)
  }
  PD_LAUNCH_CHECK("gelu_fwd_kernel");
  return PD_OK;
}

PD_EXPORT int pd_gelu_bwd(int dtype, const void* x, const void* dy, void* dx, int64_t n, int tanh_form, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x && dy && dx && n >= 0, "pd_gelu_bwd: bad arguments");
  if (n == 0) return PD_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PD_BF16 && (n % 8) == 0 && ((((uintptr_t)x) | ((uintptr_t)dy) | ((uintptr_t)dx)) & 15) == 0) {
    gelu_bwd_bf16x8_kernel<<<flat_grid(n / 8), kThreads, 0, s>>>((const uint4*)x, (const uint4*)dy, (uint4*)dx, n / 8, tanh_form);
  } else {
    PD_LN_T(dtype, gelu_bwd_kernel<T><<<flat_grid(n), kThreads, 0, s>>>((const T*)x, (const T*)dy, (T*)dx, n, tanh_form);)
  }
  PD_LAUNCH_CHECK("gelu_bwd_kernel");
  return PD_OK;
}
