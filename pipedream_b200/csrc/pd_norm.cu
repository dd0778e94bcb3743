// BatchNorm2d (training and inference) on padded-NHWC activations, for the ResNet-50 stages
// (runtime/image_classification/models/resnet50/gpus=4/stage0.py:12-55; cuDNN BN in the reference).
//
// The buffer is a [P, C] matrix, P = N*(H+2)*(W+2), whose border rows are zero; sums over all P rows are
// therefore sums over the N*H*W real pixels, and only the element count has to exclude the border.
//   forward : per-channel sum / sum of squares (two-level reduction), then y = (x-mean)*invstd*gamma+beta
//             (optional ReLU), border rows written as zero; running statistics updated like torch.
//   backward: per-channel sum(dy) and sum(dy*xhat) (ReLU mask applied first when fused), then
//             dx = gamma*invstd*(dy - sum(dy)/cnt - xhat*sum(dy*xhat)/cnt), border rows zero.
#include "pd_common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxColsPerThread = 8;      // C <= 2048

__device__ __forceinline__ bool is_border(int64_t row, int Hp, int Wp) {
  const int wp = (int)(row % Wp);
  const int hp = (int)((row / Wp) % Hp);
  return wp == 0 || wp == Wp - 1 || hp == 0 || hp == Hp - 1;
}

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

// Forward: mean, invstd from the partial sums; running statistics (momentum, unbiased variance).
__global__ void __launch_bounds__(kThreads)
bn_stats_final_kernel(const float* __restrict__ partial, int nblocks, int C, float count, float eps, float momentum,
                      float* __restrict__ mean, float* __restrict__ invstd, float* __restrict__ running_mean,
                      float* __restrict__ running_var) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f, q = 0.f;
  for (int b = 0; b < nblocks; ++b) {
    s += partial[((int64_t)b * 2) * C + c];
    q += partial[((int64_t)b * 2 + 1) * C + c];
  }
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

// Backward: sums[0][C] = sum(dy), sums[1][C] = sum(dy*xhat); also the parameter gradients.
__global__ void __launch_bounds__(kThreads)
bn_bwd_final_kernel(const float* __restrict__ partial, int nblocks, int C, float* __restrict__ sums,
                    float* __restrict__ dgamma, float* __restrict__ dbeta, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f, q = 0.f;
  for (int b = 0; b < nblocks; ++b) {
    s += partial[((int64_t)b * 2) * C + c];
    q += partial[((int64_t)b * 2 + 1) * C + c];
  }
  sums[c] = s;
  sums[C + c] = q;
  if (dbeta != nullptr) dbeta[c] = accumulate ? dbeta[c] + s : s;
  if (dgamma != nullptr) dgamma[c] = accumulate ? dgamma[c] + q : q;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
bn_apply_kernel(const T* __restrict__ x, const float* __restrict__ mean, const float* __restrict__ invstd,
                const T* __restrict__ gamma, const T* __restrict__ beta, int64_t rows, int C, int Hp, int Wp, int relu,
                T* __restrict__ y) {
  const int64_t total = rows * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const int64_t r = i / C;
    float v = 0.f;
    if (!is_border(r, Hp, Wp)) {
      v = (pd_to_float(x[i]) - mean[c]) * invstd[c] * pd_to_float(gamma[c]) + pd_to_float(beta[c]);
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
                    T* __restrict__ dx) {
  const int64_t total = rows * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const int64_t r = i / C;
    float v = 0.f;
    if (!is_border(r, Hp, Wp)) {
      float g = pd_to_float(dy[i]);
      if (y != nullptr && !(pd_to_float(y[i]) > 0.f)) g = 0.f;
      const float xhat = (pd_to_float(x[i]) - mean[c]) * invstd[c];
      v = pd_to_float(gamma[c]) * invstd[c] * (g - sums[c] * inv_count - xhat * sums[C + c] * inv_count);
    }
    dx[i] = pd_from_float<T>(v);
  }
}

int reduce_blocks() { return pd_num_sms() * 2; }
int apply_grid(int64_t total) {
  int64_t blocks = (total + kThreads - 1) / kThreads;
  int64_t cap = (int64_t)pd_num_sms() * 16;
  return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

}  // namespace

// workspace: fp32 scratch of at least pd_bn_workspace_bytes(C) bytes.
PD_EXPORT int64_t pd_bn_workspace_bytes(int C) { return (int64_t)reduce_blocks() * 2 * C * sizeof(float); }

// Training forward.  x_pad/y_pad: [N,H+2,W+2,C]; gamma/beta in `dtype`; mean/invstd: fp32 [C] (out, saved
// for backward); running_mean/var: fp32 [C], updated in place (may be NULL).
PD_EXPORT int pd_bn_fwd(int dtype, const void* x_pad, int N, int H, int W, int C, const void* gamma, const void* beta,
                        float eps, float momentum, int relu, float* mean, float* invstd, float* running_mean,
                        float* running_var, void* y_pad, void* workspace, int64_t workspace_bytes, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x_pad && gamma && beta && mean && invstd && y_pad && workspace && N > 0 && H > 0 && W > 0 && C > 0,
             "pd_bn_fwd: bad arguments");
  PD_REQUIRE(C <= kThreads * kMaxColsPerThread, "pd_bn_fwd: at most %d channels", kThreads * kMaxColsPerThread);
  PD_REQUIRE(workspace_bytes >= pd_bn_workspace_bytes(C), "pd_bn_fwd: workspace too small");
  cudaStream_t s = (cudaStream_t)stream;
  const int Hp = H + 2, Wp = W + 2;
  const int64_t rows = (int64_t)N * Hp * Wp;
  const int nb = reduce_blocks();
  const float count = (float)((int64_t)N * H * W);
  if (dtype == PD_F32)
    bn_reduce_kernel<float><<<nb, kThreads, 0, s>>>((const float*)x_pad, nullptr, nullptr, nullptr, nullptr, rows, C, 0, (float*)workspace);
  else if (dtype == PD_BF16)
    bn_reduce_kernel<__nv_bfloat16><<<nb, kThreads, 0, s>>>((const __nv_bfloat16*)x_pad, nullptr, nullptr, nullptr, nullptr, rows, C, 0, (float*)workspace);
  else PD_REQUIRE(false, "pd_bn_fwd: bad dtype");
  PD_LAUNCH_CHECK("bn_reduce_kernel");
  bn_stats_final_kernel<<<(C + kThreads - 1) / kThreads, kThreads, 0, s>>>((const float*)workspace, nb, C, count, eps, momentum,
                                                                           mean, invstd, running_mean, running_var);
  PD_LAUNCH_CHECK("bn_stats_final_kernel");
  const int grid = apply_grid(rows * C);
  if (dtype == PD_F32)
    bn_apply_kernel<float><<<grid, kThreads, 0, s>>>((const float*)x_pad, mean, invstd, (const float*)gamma, (const float*)beta,
                                                     rows, C, Hp, Wp, relu, (float*)y_pad);
  else
    bn_apply_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)x_pad, mean, invstd, (const __nv_bfloat16*)gamma,
                                                             (const __nv_bfloat16*)beta, rows, C, Hp, Wp, relu, (__nv_bfloat16*)y_pad);
  PD_LAUNCH_CHECK("bn_apply_kernel");
  return PD_OK;
}

// Inference forward: normalises with the given statistics (mean, invstd fp32 [C]).
PD_EXPORT int pd_bn_apply(int dtype, const void* x_pad, int N, int H, int W, int C, const void* gamma, const void* beta,
                          const float* mean, const float* invstd, int relu, void* y_pad, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x_pad && gamma && beta && mean && invstd && y_pad && N > 0 && H > 0 && W > 0 && C > 0, "pd_bn_apply: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  const int Hp = H + 2, Wp = W + 2;
  const int64_t rows = (int64_t)N * Hp * Wp;
  const int grid = apply_grid(rows * C);
  if (dtype == PD_F32)
    bn_apply_kernel<float><<<grid, kThreads, 0, s>>>((const float*)x_pad, mean, invstd, (const float*)gamma, (const float*)beta,
                                                     rows, C, Hp, Wp, relu, (float*)y_pad);
  else if (dtype == PD_BF16)
    bn_apply_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)x_pad, mean, invstd, (const __nv_bfloat16*)gamma,
                                                             (const __nv_bfloat16*)beta, rows, C, Hp, Wp, relu, (__nv_bfloat16*)y_pad);
  else PD_REQUIRE(false, "pd_bn_apply: bad dtype");
  PD_LAUNCH_CHECK("bn_apply_kernel");
  return PD_OK;
}

// Training backward.  y_pad != NULL: the forward fused a ReLU and dy is masked by (y > 0) first.
// dgamma/dbeta: fp32 [C] (stored, or added to when accumulate != 0).  sums_ws: fp32 [2*C] scratch.
PD_EXPORT int pd_bn_bwd(int dtype, const void* x_pad, const void* dy_pad, const void* y_pad, int N, int H, int W, int C,
                        const void* gamma, const float* mean, const float* invstd, float* dgamma, float* dbeta,
                        int accumulate, void* dx_pad, float* sums_ws, void* workspace, int64_t workspace_bytes,
                        void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x_pad && dy_pad && gamma && mean && invstd && dx_pad && sums_ws && workspace && N > 0 && H > 0 && W > 0 && C > 0,
             "pd_bn_bwd: bad arguments");
  PD_REQUIRE(C <= kThreads * kMaxColsPerThread, "pd_bn_bwd: at most %d channels", kThreads * kMaxColsPerThread);
  PD_REQUIRE(workspace_bytes >= pd_bn_workspace_bytes(C), "pd_bn_bwd: workspace too small");
  cudaStream_t s = (cudaStream_t)stream;
  const int Hp = H + 2, Wp = W + 2;
  const int64_t rows = (int64_t)N * Hp * Wp;
  const int nb = reduce_blocks();
  const float inv_count = 1.f / (float)((int64_t)N * H * W);
  if (dtype == PD_F32)
    bn_reduce_kernel<float><<<nb, kThreads, 0, s>>>((const float*)x_pad, (const float*)dy_pad, (const float*)y_pad, mean, invstd, rows, C, 1, (float*)workspace);
  else if (dtype == PD_BF16)
    bn_reduce_kernel<__nv_bfloat16><<<nb, kThreads, 0, s>>>((const __nv_bfloat16*)x_pad, (const __nv_bfloat16*)dy_pad,
                                                            (const __nv_bfloat16*)y_pad, mean, invstd, rows, C, 1, (float*)workspace);
  else PD_REQUIRE(false, "pd_bn_bwd: bad dtype");
  PD_LAUNCH_CHECK("bn_reduce_kernel");
  bn_bwd_final_kernel<<<(C + kThreads - 1) / kThreads, kThreads, 0, s>>>((const float*)workspace, nb, C, sums_ws, dgamma, dbeta, accumulate);
  PD_LAUNCH_CHECK("bn_bwd_final_kernel");
  const int grid = apply_grid(rows * C);
  if (dtype == PD_F32)
    bn_bwd_apply_kernel<float><<<grid, kThreads, 0, s>>>((const float*)x_pad, (const float*)dy_pad, (const float*)y_pad, mean, invstd,
                                                         (const float*)gamma, sums_ws, rows, C, Hp, Wp, inv_count, (float*)dx_pad);
  else
    bn_bwd_apply_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)x_pad, (const __nv_bfloat16*)dy_pad,
                                                                 (const __nv_bfloat16*)y_pad, mean, invstd, (const __nv_bfloat16*)gamma,
                                                                 sums_ws, rows, C, Hp, Wp, inv_count, (__nv_bfloat16*)dx_pad);
  PD_LAUNCH_CHECK("bn_bwd_apply_kernel");
  return PD_OK;
}
