// BatchNorm2d (training and inference) on padded-NHWC activations, for the ResNet-50 stages
// (runtime/image_classification/models/resnet50/gpus=4/stage0.py:12-55; cuDNN BN in the reference),
// with the residual add and the ReLU that follow the last normalisation of a bottleneck block
// (stage1.py forward: `out = out + identity; out = relu(out)`) folded into the same passes.
//
// The buffer is a [P, C] matrix, P = N*(H+2)*(W+2), whose border rows are zero; sums over all P rows are
// therefore sums over the N*H*W real pixels, and only the element count has to exclude the border.
//   forward : per-channel sum / sum of squares (two-level reduction, fixed order: deterministic), then
//             y = (x-mean)*invstd*gamma+beta (+ residual) (optional ReLU), border rows written as zero;
//             running statistics updated like torch.
//   backward: g = dy (zeroed where y <= 0 when the forward applied a ReLU); per-channel sum(g) and
//             sum(g*xhat); dx = gamma*invstd*(g - sum(g)/cnt - xhat*sum(g*xhat)/cnt), border rows zero;
//             g itself is the gradient of the residual input.
// All kernels are HBM-bound: bf16 tensors whose channel count is a multiple of 8 with C/8 dividing 256
// (every ResNet-50 layer) take a path with 16-byte accesses in which a thread keeps the same 8 channels
// for the whole launch; everything else takes the generic scalar path.
#include "pd_common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxColsPerThread = 8;      // generic path: C <= 2048

__device__ __forceinline__ bool is_border(int64_t row, int Hp, int Wp) {
  const int wp = (int)(row % Wp);
  const int hp = (int)((row / Wp) % Hp);
  return wp == 0 || wp == Wp - 1 || hp == 0 || hp == Hp - 1;
}

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

// ------------------------------------------------------------------------------------------------
// generic path (fp32, or channel counts the vector path does not take)
// ------------------------------------------------------------------------------------------------
// partial[block][0][C] = sum_r a(r,c), partial[block][1][C] = sum_r b(r,c) over the block's rows.
//   mode 0 (forward statistics): a = x, b = x*x
//   mode 1 (backward sums)     : g = dy (zeroed where y <= 0 when y != null); a = g, b = g * xhat
template <typename T>
__global__ void __launch_bounds__(kThreads)
bn_reduce_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ y,
                 const float* __restrict__ mean, const float* __restrict__ invstd, int64_t rows, int C, int mode,
                 float* __restrict__ partial) {
  float a[kMaxColsPerThread], b[kMaxColsPerThread];
#pragma unroll
  for (int k = 0; k < kMaxColsPerThread; ++k) a[k] = b[k] = 0.f;
  const int64_t per = (rows + gridDim.x - 1) / gridDim.x;
  const int64_t r0 = (int64_t)blockIdx.x * per, r1 = min(rows, r0 + per);
  for (int64_t r = r0; r < r1; ++r) {
#pragma unroll
    for (int k = 0; k < kMaxColsPerThread; ++k) {
      const int c = threadIdx.x + k * kThreads;
      if (c < C) {
        const int64_t i = r * C + c;
        if (mode == 0) {
          const float v = pd_to_float(x[i]);
          a[k] += v; b[k] += v * v;
        } else {
          float g = pd_to_float(dy[i]);
          if (y != nullptr && !(pd_to_float(y[i]) > 0.f)) g = 0.f;
          a[k] += g;
          b[k] += g * (pd_to_float(x[i]) - mean[c]) * invstd[c];
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < kMaxColsPerThread; ++k) {
    const int c = threadIdx.x + k * kThreads;
    if (c < C) {
      partial[((int64_t)blockIdx.x * 2) * C + c] = a[k];
      partial[((int64_t)blockIdx.x * 2 + 1) * C + c] = b[k];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
bn_apply_kernel(const T* __restrict__ x, const T* __restrict__ res, const float* __restrict__ mean,
                const float* __restrict__ invstd, const T* __restrict__ gamma, const T* __restrict__ beta,
                int64_t rows, int C, int Hp, int Wp, int relu, T* __restrict__ y) {
  const int64_t total = rows * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const int64_t r = i / C;
    float v = 0.f;
    if (!is_border(r, Hp, Wp)) {
      v = (pd_to_float(x[i]) - mean[c]) * invstd[c] * pd_to_float(gamma[c]) + pd_to_float(beta[c]);
      if (res != nullptr) v += pd_to_float(res[i]);
      if (relu) v = fmaxf(v, 0.f);
    }
    y[i] = pd_from_float<T>(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
bn_bwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ y,
                    const float* __restrict__ mean, const float* __restrict__ invstd, const T* __restrict__ gamma,
                    const float* __restrict__ sums, int64_t rows, int C, int Hp, int Wp, float inv_count,
                    T* __restrict__ dx, T* __restrict__ dres) {
  const int64_t total = rows * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const int64_t r = i / C;
    float v = 0.f, g = 0.f;
    if (!is_border(r, Hp, Wp)) {
      g = pd_to_float(dy[i]);
      if (y != nullptr && !(pd_to_float(y[i]) > 0.f)) g = 0.f;
      const float xhat = (pd_to_float(x[i]) - mean[c]) * invstd[c];
      v = pd_to_float(gamma[c]) * invstd[c] * (g - sums[c] * inv_count - xhat * sums[C + c] * inv_count);
    }
    dx[i] = pd_from_float<T>(v);
    if (dres != nullptr) dres[i] = pd_from_float<T>(g);
  }
}

// ------------------------------------------------------------------------------------------------
// second level of the reductions (both paths): one block per 32 channels, 32 slices of the partials each
// (the loop over the partials is a chain of L2 round trips: short and wide beats long and narrow)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void sum_partials(const float* __restrict__ partial, int nblocks, int C, int c,
                                             float (*sh)[32][33], float& s, float& q) {
  s = q = 0.f;
  if (c < C) {
#pragma unroll 4
    for (int b = threadIdx.y; b < nblocks; b += 32) {
      s += partial[((int64_t)b * 2) * C + c];
      q += partial[((int64_t)b * 2 + 1) * C + c];
    }
  }
  sh[0][threadIdx.y][threadIdx.x] = s;
  sh[1][threadIdx.y][threadIdx.x] = q;
  __syncthreads();
  if (threadIdx.y == 0) {
    s = q = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      s += sh[0][j][threadIdx.x];
      q += sh[1][j][threadIdx.x];
    }
  }
}

// Forward: mean, invstd from the partial sums; running statistics (momentum, unbiased variance).
__global__ void __launch_bounds__(1024)
bn_stats_final_kernel(const float* __restrict__ partial, int nblocks, int C, float count, float eps, float momentum,
                      float* __restrict__ mean, float* __restrict__ invstd, float* __restrict__ running_mean,
                      float* __restrict__ running_var) {
  __shared__ float sh[2][32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s, q;
  sum_partials(partial, nblocks, C, c, sh, s, q);
  if (threadIdx.y != 0 || c >= C) return;
  const float m = s / count;
  const float var = fmaxf(q / count - m * m, 0.f);
  mean[c] = m;
  invstd[c] = rsqrtf(var + eps);
  if (running_mean != nullptr) {
    running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * m;
    const float unbiased = count > 1.f ? var * count / (count - 1.f) : var;
    running_var[c] = (1.f - momentum) * running_var[c] + momentum * unbiased;
  }
}

// Backward: sums[0][C] = sum(g), sums[1][C] = sum(g*xhat); also the parameter gradients.
__global__ void __launch_bounds__(1024)
bn_bwd_final_kernel(const float* __restrict__ partial, int nblocks, int C, float* __restrict__ sums,
                    float* __restrict__ dgamma, float* __restrict__ dbeta, int accumulate) {
  __shared__ float sh[2][32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s, q;
  sum_partials(partial, nblocks, C, c, sh, s, q);
  if (threadIdx.y != 0 || c >= C) return;
  sums[c] = s;
  sums[C + c] = q;
  if (dbeta != nullptr) dbeta[c] = accumulate ? dbeta[c] + s : s;
  if (dgamma != nullptr) dgamma[c] = accumulate ? dgamma[c] + q : q;
}

// ------------------------------------------------------------------------------------------------
// bf16 vector path.  The matrix is read as nvec = P*C/8 16-byte vectors; G = C/8 vectors per row,
// G a power of two <= 256, so a thread's channel group (index mod G) never changes.
// ------------------------------------------------------------------------------------------------
template <int MODE, bool MASK>
__global__ void __launch_bounds__(kThreads)
bn_reduce_v8_kernel(const uint4* __restrict__ x, const uint4* __restrict__ dy, const uint4* __restrict__ y,
                    const float* __restrict__ mean, const float* __restrict__ invstd, int64_t nvec, int G, int C,
                    float* __restrict__ partial) {
  __shared__ float sh[kThreads][17];
  const int tid = threadIdx.x;
  const int cg = tid & (G - 1);
  float a[8], b[8], m[8], is[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    a[k] = b[k] = 0.f;
    if (MODE == 1) { m[k] = mean[cg * 8 + k]; is[k] = invstd[cg * 8 + k]; }
  }
  // contiguous chunk per block, a multiple of the block size so that the channel group stays put
  const int64_t per = (((nvec + gridDim.x - 1) / gridDim.x) + kThreads - 1) / kThreads * kThreads;
  const int64_t v0 = (int64_t)blockIdx.x * per;
  const int64_t v1 = min(nvec, v0 + per);
  constexpr int U = MODE == 0 ? 4 : 2;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (int64_t base = v0 + tid; base < v1; base += (int64_t)kThreads * U) {
    uint4 xv[U], gv[U], yv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = base + (int64_t)u * kThreads;
      const bool ok = i < v1;
      xv[u] = ok ? x[i] : zero;
      if (MODE == 1) gv[u] = ok ? dy[i] : zero;
      if (MODE == 1 && MASK) yv[u] = ok ? y[i] : zero;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float xf[8];
      unpack8(xv[u], xf);
      if (MODE == 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) { a[k] += xf[k]; b[k] += xf[k] * xf[k]; }
      } else {
        float gf[8], yf[8];
        unpack8(gv[u], gf);
        if (MASK) unpack8(yv[u], yf);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float g = gf[k];
          if (MASK && !(yf[k] > 0.f)) g = 0.f;
          a[k] += g;
          b[k] += g * (xf[k] - m[k]) * is[k];
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) { sh[tid][k] = a[k]; sh[tid][8 + k] = b[k]; }
  __syncthreads();
  const int R = kThreads / G;
  for (int j = tid; j < 16 * G; j += kThreads) {
    const int g2 = j & (G - 1), k = j / G;
    float s = 0.f;
    for (int r = 0; r < R; ++r) s += sh[r * G + g2][k];
    partial[((int64_t)blockIdx.x * 2 + (k >> 3)) * C + g2 * 8 + (k & 7)] = s;
  }
}

__device__ __forceinline__ bool border_of_vec(int64_t i, int gshift, int Hp, int Wp) {
  const unsigned row = (unsigned)(i >> gshift);
  const unsigned q = row / (unsigned)Wp;
  const unsigned wp = row - q * (unsigned)Wp;
  const unsigned hp = q % (unsigned)Hp;
  return wp == 0 || wp == (unsigned)Wp - 1 || hp == 0 || hp == (unsigned)Hp - 1;
}

__global__ void __launch_bounds__(kThreads)
bn_apply_v8_kernel(const uint4* __restrict__ x, const uint4* __restrict__ res, const float* __restrict__ mean,
                   const float* __restrict__ invstd, const __nv_bfloat16* __restrict__ gamma,
                   const __nv_bfloat16* __restrict__ beta, int64_t nvec, int G, int gshift, int Hp, int Wp, int relu,
                   uint4* __restrict__ y) {
  const int cg = threadIdx.x & (G - 1);
  float scale[8], shift[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int c = cg * 8 + k;
    scale[k] = invstd[c] * __bfloat162float(gamma[c]);
    shift[k] = __bfloat162float(beta[c]) - mean[c] * scale[k];
  }
  constexpr int U = 4;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (int64_t base = (int64_t)blockIdx.x * kThreads + threadIdx.x; base < nvec; base += stride * U) {
    uint4 xv[U], rv[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = base + (int64_t)u * stride;
      ok[u] = i < nvec && !border_of_vec(i, gshift, Hp, Wp);
      xv[u] = ok[u] ? x[i] : zero;
      if (res != nullptr) rv[u] = ok[u] ? res[i] : zero;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = base + (int64_t)u * stride;
      if (i >= nvec) break;
      uint4 out = zero;
      if (ok[u]) {
        float f[8], r[8];
        unpack8(xv[u], f);
        if (res != nullptr) unpack8(rv[u], r);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float v = f[k] * scale[k] + shift[k];
          if (res != nullptr) v += r[k];
          f[k] = relu ? fmaxf(v, 0.f) : v;
        }
        out = pack8(f);
      }
      y[i] = out;
    }
  }
}

template <bool MASK>
__global__ void __launch_bounds__(kThreads)
bn_bwd_apply_v8_kernel(const uint4* __restrict__ x, const uint4* __restrict__ dy, const uint4* __restrict__ y,
                       const float* __restrict__ mean, const float* __restrict__ invstd,
                       const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ sums, int64_t nvec, int G,
                       int gshift, int C, int Hp, int Wp, float inv_count, uint4* __restrict__ dx,
                       uint4* __restrict__ dres) {
  const int cg = threadIdx.x & (G - 1);
  // dx = k1 * (g - c1 - (x - mean) * c2),  k1 = gamma*invstd, c1 = sum(g)/cnt, c2 = invstd*sum(g*xhat)/cnt
  float k1[8], c1[8], c2[8], m[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int c = cg * 8 + k;
    const float is = invstd[c];
    k1[k] = __bfloat162float(gamma[c]) * is;
    c1[k] = sums[c] * inv_count;
    c2[k] = is * sums[C + c] * inv_count;
    m[k] = mean[c];
  }
  constexpr int U = 2;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (int64_t base = (int64_t)blockIdx.x * kThreads + threadIdx.x; base < nvec; base += stride * U) {
    uint4 xv[U], gv[U], yv[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = base + (int64_t)u * stride;
      ok[u] = i < nvec && !border_of_vec(i, gshift, Hp, Wp);
      xv[u] = ok[u] ? x[i] : zero;
      gv[u] = ok[u] ? dy[i] : zero;
      if (MASK) yv[u] = ok[u] ? y[i] : zero;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = base + (int64_t)u * stride;
      if (i >= nvec) break;
      uint4 out = zero, gout = zero;
      if (ok[u]) {
        float xf[8], gf[8], yf[8];
        unpack8(xv[u], xf);
        unpack8(gv[u], gf);
        if (MASK) unpack8(yv[u], yf);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (MASK && !(yf[k] > 0.f)) gf[k] = 0.f;
          xf[k] = k1[k] * (gf[k] - c1[k] - (xf[k] - m[k]) * c2[k]);
        }
        out = pack8(xf);
        if (dres != nullptr) gout = pack8(gf);
      }
      dx[i] = out;
      if (dres != nullptr) dres[i] = gout;
    }
  }
}

int reduce_blocks() { return pd_num_sms() * 4; }
int apply_grid(int64_t total) {
  int64_t blocks = (total + kThreads - 1) / kThreads;
  int64_t cap = (int64_t)pd_num_sms() * 16;
  return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}
// vector path: grid capped at 8 blocks per SM, `per_thread` vectors per thread and pass
int vec_grid(int64_t nvec, int per_thread) {
  int64_t blocks = (nvec + (int64_t)kThreads * per_thread - 1) / ((int64_t)kThreads * per_thread);
  int64_t cap = (int64_t)pd_num_sms() * 8;
  return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}
// number of first-level blocks: one per 64 KB of input, at most reduce_blocks()
int reduce_grid(int64_t nvec) {
  int64_t blocks = (nvec * 16 + 65535) / 65536;
  int64_t cap = reduce_blocks();
  return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}
bool vector_path(int dtype, int C) {
  if (dtype != PD_BF16 || (C % 8) != 0) return false;
  const int G = C / 8;
  return G <= kThreads && (G & (G - 1)) == 0;
}
int log2i(int v) { int s = 0; while ((1 << s) < v) ++s; return s; }

}  // namespace

// workspace: fp32 scratch of at least pd_bn_workspace_bytes(C) bytes.
PD_EXPORT int64_t pd_bn_workspace_bytes(int C) { return (int64_t)reduce_blocks() * 2 * C * sizeof(float); }

// Training forward.  x_pad/y_pad (and res_pad, the optional tensor added before the ReLU): [N,H+2,W+2,C];
// gamma/beta in `dtype`; mean/invstd: fp32 [C] (out, saved for backward); running_mean/var: fp32 [C],
// updated in place (may be NULL).
PD_EXPORT int pd_bn_fwd(int dtype, const void* x_pad, const void* res_pad, int N, int H, int W, int C, const void* gamma,
                        const void* beta, float eps, float momentum, int relu, float* mean, float* invstd,
                        float* running_mean, float* running_var, void* y_pad, void* workspace, int64_t workspace_bytes,
                        void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x_pad && gamma && beta && mean && invstd && y_pad && workspace && N > 0 && H > 0 && W > 0 && C > 0,
             "pd_bn_fwd: bad arguments");
  PD_REQUIRE(dtype == PD_F32 || dtype == PD_BF16, "pd_bn_fwd: bad dtype");
  PD_REQUIRE(C <= kThreads * kMaxColsPerThread, "pd_bn_fwd: at most %d channels", kThreads * kMaxColsPerThread);
  PD_REQUIRE(workspace_bytes >= pd_bn_workspace_bytes(C), "pd_bn_fwd: workspace too small");
  cudaStream_t s = (cudaStream_t)stream;
  const int Hp = H + 2, Wp = W + 2;
  const int64_t rows = (int64_t)N * Hp * Wp;
  PD_REQUIRE(rows < (1ll << 31), "pd_bn_fwd: too many rows");
  const float count = (float)((int64_t)N * H * W);
  const bool vec = vector_path(dtype, C);
  const int64_t nvec = rows * C / 8;
  int nb;
  if (vec) {
    nb = reduce_grid(nvec);
    bn_reduce_v8_kernel<0, false><<<nb, kThreads, 0, s>>>((const uint4*)x_pad, nullptr, nullptr, nullptr, nullptr, nvec,
                                                          C / 8, C, (float*)workspace);
  } else {
    nb = reduce_blocks();
    if (dtype == PD_F32)
      bn_reduce_kernel<float><<<nb, kThreads, 0, s>>>((const float*)x_pad, nullptr, nullptr, nullptr, nullptr, rows, C, 0, (float*)workspace);
    else
      bn_reduce_kernel<__nv_bfloat16><<<nb, kThreads, 0, s>>>((const __nv_bfloat16*)x_pad, nullptr, nullptr, nullptr, nullptr, rows, C, 0, (float*)workspace);
  }
  PD_LAUNCH_CHECK("bn_reduce_kernel");
  bn_stats_final_kernel<<<(C + 31) / 32, dim3(32, 32), 0, s>>>((const float*)workspace, nb, C, count, eps, momentum,
                                                              mean, invstd, running_mean, running_var);
  PD_LAUNCH_CHECK("bn_stats_final_kernel");
  if (vec) {
    bn_apply_v8_kernel<<<vec_grid(nvec, 4), kThreads, 0, s>>>((const uint4*)x_pad, (const uint4*)res_pad, mean, invstd,
                                                               (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)beta, nvec,
                                                               C / 8, log2i(C / 8), Hp, Wp, relu, (uint4*)y_pad);
  } else {
    const int grid = apply_grid(rows * C);
    if (dtype == PD_F32)
      bn_apply_kernel<float><<<grid, kThreads, 0, s>>>((const float*)x_pad, (const float*)res_pad, mean, invstd, (const float*)gamma,
                                                       (const float*)beta, rows, C, Hp, Wp, relu, (float*)y_pad);
    else
      bn_apply_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)x_pad, (const __nv_bfloat16*)res_pad, mean, invstd,
                                                               (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)beta, rows, C, Hp, Wp,
                                                               relu, (__nv_bfloat16*)y_pad);
  }
  PD_LAUNCH_CHECK("bn_apply_kernel");
  return PD_OK;
}

// Inference forward: normalises with the given statistics (mean, invstd fp32 [C]).
PD_EXPORT int pd_bn_apply(int dtype, const void* x_pad, const void* res_pad, int N, int H, int W, int C, const void* gamma,
                          const void* beta, const float* mean, const float* invstd, int relu, void* y_pad, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x_pad && gamma && beta && mean && invstd && y_pad && N > 0 && H > 0 && W > 0 && C > 0, "pd_bn_apply: bad arguments");
  PD_REQUIRE(dtype == PD_F32 || dtype == PD_BF16, "pd_bn_apply: bad dtype");
  cudaStream_t s = (cudaStream_t)stream;
  const int Hp = H + 2, Wp = W + 2;
  const int64_t rows = (int64_t)N * Hp * Wp;
  PD_REQUIRE(rows < (1ll << 31), "pd_bn_apply: too many rows");
  if (vector_path(dtype, C)) {
    const int64_t nvec = rows * C / 8;
    bn_apply_v8_kernel<<<vec_grid(nvec, 4), kThreads, 0, s>>>((const uint4*)x_pad, (const uint4*)res_pad, mean, invstd,
                                                               (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)beta, nvec,
                                                               C / 8, log2i(C / 8), Hp, Wp, relu, (uint4*)y_pad);
  } else {
    const int grid = apply_grid(rows * C);
    if (dtype == PD_F32)
      bn_apply_kernel<float><<<grid, kThreads, 0, s>>>((const float*)x_pad, (const float*)res_pad, mean, invstd, (const float*)gamma,
                                                       (const float*)beta, rows, C, Hp, Wp, relu, (float*)y_pad);
    else
      bn_apply_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)x_pad, (const __nv_bfloat16*)res_pad, mean, invstd,
                                                               (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)beta, rows, C, Hp, Wp,
                                                               relu, (__nv_bfloat16*)y_pad);
  }
  PD_LAUNCH_CHECK("bn_apply_kernel");
  return PD_OK;
}

// Training backward.  y_pad != NULL: the forward applied a ReLU and dy is masked by (y > 0) first.
// dgamma/dbeta: fp32 [C] (stored, or added to when accumulate != 0).  dres_pad (may be NULL): receives
// the masked dy, i.e. the gradient of the residual input.  sums_ws: fp32 [2*C] scratch.
PD_EXPORT int pd_bn_bwd(int dtype, const void* x_pad, const void* dy_pad, const void* y_pad, int N, int H, int W, int C,
                        const void* gamma, const float* mean, const float* invstd, float* dgamma, float* dbeta,
                        int accumulate, void* dx_pad, void* dres_pad, float* sums_ws, void* workspace,
                        int64_t workspace_bytes, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x_pad && dy_pad && gamma && mean && invstd && dx_pad && sums_ws && workspace && N > 0 && H > 0 && W > 0 && C > 0,
             "pd_bn_bwd: bad arguments");
  PD_REQUIRE(dtype == PD_F32 || dtype == PD_BF16, "pd_bn_bwd: bad dtype");
  PD_REQUIRE(C <= kThreads * kMaxColsPerThread, "pd_bn_bwd: at most %d channels", kThreads * kMaxColsPerThread);
  PD_REQUIRE(workspace_bytes >= pd_bn_workspace_bytes(C), "pd_bn_bwd: workspace too small");
  cudaStream_t s = (cudaStream_t)stream;
  const int Hp = H + 2, Wp = W + 2;
  const int64_t rows = (int64_t)N * Hp * Wp;
  PD_REQUIRE(rows < (1ll << 31), "pd_bn_bwd: too many rows");
  const float inv_count = 1.f / (float)((int64_t)N * H * W);
  const bool vec = vector_path(dtype, C);
  const int64_t nvec = rows * C / 8;
  int nb;
  if (vec) {
    nb = reduce_grid(nvec);
    if (y_pad != nullptr)
      bn_reduce_v8_kernel<1, true><<<nb, kThreads, 0, s>>>((const uint4*)x_pad, (const uint4*)dy_pad, (const uint4*)y_pad, mean,
                                                           invstd, nvec, C / 8, C, (float*)workspace);
    else
      bn_reduce_v8_kernel<1, false><<<nb, kThreads, 0, s>>>((const uint4*)x_pad, (const uint4*)dy_pad, nullptr, mean, invstd, nvec,
                                                            C / 8, C, (float*)workspace);
  } else {
    nb = reduce_blocks();
    if (dtype == PD_F32)
      bn_reduce_kernel<float><<<nb, kThreads, 0, s>>>((const float*)x_pad, (const float*)dy_pad, (const float*)y_pad, mean, invstd, rows, C, 1, (float*)workspace);
    else
      bn_reduce_kernel<__nv_bfloat16><<<nb, kThreads, 0, s>>>((const __nv_bfloat16*)x_pad, (const __nv_bfloat16*)dy_pad,
                                                              (const __nv_bfloat16*)y_pad, mean, invstd, rows, C, 1, (float*)workspace);
  }
  PD_LAUNCH_CHECK("bn_reduce_kernel");
  bn_bwd_final_kernel<<<(C + 31) / 32, dim3(32, 32), 0, s>>>((const float*)workspace, nb, C, sums_ws, dgamma, dbeta, accumulate);
  PD_LAUNCH_CHECK("bn_bwd_final_kernel");
  if (vec) {
    const int grid = vec_grid(nvec, 2);
    if (y_pad != nullptr)
      bn_bwd_apply_v8_kernel<true><<<grid, kThreads, 0, s>>>((const uint4*)x_pad, (const uint4*)dy_pad, (const uint4*)y_pad, mean, invstd,
                                                             (const __nv_bfloat16*)gamma, sums_ws, nvec, C / 8, log2i(C / 8), C, Hp, Wp,
                                                             inv_count, (uint4*)dx_pad, (uint4*)dres_pad);
    else
      bn_bwd_apply_v8_kernel<false><<<grid, kThreads, 0, s>>>((const uint4*)x_pad, (const uint4*)dy_pad, nullptr, mean, invstd,
                                                              (const __nv_bfloat16*)gamma, sums_ws, nvec, C / 8, log2i(C / 8), C, Hp, Wp,
                                                              inv_count, (uint4*)dx_pad, (uint4*)dres_pad);
  } else {
    const int grid = apply_grid(rows * C);
    if (dtype == PD_F32)
      bn_bwd_apply_kernel<float><<<grid, kThreads, 0, s>>>((const float*)x_pad, (const float*)dy_pad, (const float*)y_pad, mean, invstd,
                                                           (const float*)gamma, sums_ws, rows, C, Hp, Wp, inv_count, (float*)dx_pad,
                                                           (float*)dres_pad);
    else
      bn_bwd_apply_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)x_pad, (const __nv_bfloat16*)dy_pad,
                                                                   (const __nv_bfloat16*)y_pad, mean, invstd, (const __nv_bfloat16*)gamma,
                                                                   sums_ws, rows, C, Hp, Wp, inv_count, (__nv_bfloat16*)dx_pad,
                                                                   (__nv_bfloat16*)dres_pad);
  }
  PD_LAUNCH_CHECK("bn_bwd_apply_kernel");
  return PD_OK;
}
