// Fused optimizer step over the stage's weight-version ring.
//
// All parameters of a pipeline stage live in one flat arena of `num_slots`
// versions ("slots") of `n` elements each.  One launch reads the gradient, the
// newest weights (fp32 master when the compute copy is bf16) and the optimizer
// state, and writes the updated weights into the slot that held the oldest
// version.  This replaces the per-tensor torch.optim loop plus the three
// full-model copies per minibatch of the reference wrapper
// (runtime/optimizer.py:64-116,122-164).
#include "pd_common.cuh"

namespace {

constexpr int kOptThreads = 256;

// Four consecutive weights as one store (16 bytes of fp32, 8 bytes of bf16); `dst` is aligned to that size.
__device__ __forceinline__ void store4(float* dst, const float* p) {
  *reinterpret_cast<float4*>(dst) = make_float4(p[0], p[1], p[2], p[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, const float* p) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(p[0], p[1]), hi = __floats2bfloat162_rn(p[2], p[3]);
  uint2 v;
  v.x = *reinterpret_cast<uint32_t*>(&lo);
  v.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = v;
}

template <typename WT>
__global__ void __launch_bounds__(kOptThreads)
sgd_ring_kernel(const WT* __restrict__ w_read, WT* __restrict__ w_write,
                float* __restrict__ master, const float* __restrict__ grad,
                float* __restrict__ mom, int64_t n, float lr, float momentum,
                float dampening, float wd, int nesterov, int first_step,
                float grad_scale) {
  // 4 elements per thread per iteration; arena offsets are 16-byte aligned.
  int64_t i4 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const bool vec = ((((uintptr_t)grad) | ((uintptr_t)mom) | ((uintptr_t)master)) & 15) == 0 &&
                   ((((uintptr_t)w_read) | ((uintptr_t)w_write)) & (4 * sizeof(WT) - 1)) == 0;
  const int64_t n4 = vec ? n >> 2 : 0;
  for (; i4 < n4; i4 += stride) {
    const int64_t i = i4 << 2;
    float4 g = *reinterpret_cast<const float4*>(grad + i);
    float p[4];
    if (master != nullptr) {
      float4 m4 = *reinterpret_cast<const float4*>(master + i);
      p[0] = m4.x; p[1] = m4.y; p[2] = m4.z; p[3] = m4.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) p[j] = pd_to_float(w_read[i + j]);
    }
    float gg[4] = {g.x * grad_scale, g.y * grad_scale, g.z * grad_scale, g.w * grad_scale};
    float b[4] = {0.f, 0.f, 0.f, 0.f};
    if (momentum != 0.f && !first_step) {
      float4 b4 = *reinterpret_cast<const float4*>(mom + i);
      b[0] = b4.x; b[1] = b4.y; b[2] = b4.z; b[3] = b4.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float d = gg[j];
      if (wd != 0.f) d = fmaf(wd, p[j], d);
      if (momentum != 0.f) {
        if (first_step) b[j] = d;
        else b[j] = fmaf(momentum, b[j], (1.f - dampening) * d);
        d = nesterov ? fmaf(momentum, b[j], d) : b[j];
      }
      p[j] = fmaf(-lr, d, p[j]);
    }
    if (momentum != 0.f)
      *reinterpret_cast<float4*>(mom + i) = make_float4(b[0], b[1], b[2], b[3]);
    if (master != nullptr)
      *reinterpret_cast<float4*>(master + i) = make_float4(p[0], p[1], p[2], p[3]);
    store4(w_write + i, p);
  }
  // tail (n not a multiple of 4), or everything when the pointers are not aligned
  for (int64_t t = (n4 << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += stride) {
    float pj = master ? master[t] : pd_to_float(w_read[t]);
    float d = grad[t] * grad_scale;
    if (wd != 0.f) d = fmaf(wd, pj, d);
    if (momentum != 0.f) {
      float bj = first_step ? d : fmaf(momentum, mom[t], (1.f - dampening) * d);
      mom[t] = bj;
      d = nesterov ? fmaf(momentum, bj, d) : bj;
    }
    pj = fmaf(-lr, d, pj);
    if (master) master[t] = pj;
    w_write[t] = pd_from_float<WT>(pj);
  }
}

__device__ __forceinline__ void adam_update(float& p, float g, float& m, float& v, float beta1, float beta2, float eps,
                                            float wd, float step_size, float bias_c2_sqrt) {
  if (wd != 0.f) g = fmaf(wd, p, g);
  m = m + (g - m) * (1.f - beta1);           // lerp form used by torch.optim.Adam
  v = v * beta2 + (1.f - beta2) * g * g;
  const float denom = sqrtf(v) / bias_c2_sqrt + eps;
  p = p - step_size * (m / denom);
}

// Four parameters per thread and trip: 16-byte loads and stores of gradient, moments and master copy (every arena
// is 256-byte aligned and slot strides are multiples of 64 elements), one 8-byte store of the bf16 weights.
template <typename WT>
__global__ void __launch_bounds__(kOptThreads)
adam_ring_kernel(const WT* __restrict__ w_read, WT* __restrict__ w_write,
                 float* __restrict__ master, const float* __restrict__ grad,
                 float* __restrict__ exp_avg, float* __restrict__ exp_avg_sq,
                 int64_t n, float lr, float beta1, float beta2, float eps, float wd,
                 float bias_c1, float bias_c2_sqrt, float grad_scale) {
  const float step_size = lr / bias_c1;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const bool vec = ((((uintptr_t)grad) | ((uintptr_t)exp_avg) | ((uintptr_t)exp_avg_sq) | ((uintptr_t)master)) & 15) == 0 &&
                   ((((uintptr_t)w_read) | ((uintptr_t)w_write)) & (4 * sizeof(WT) - 1)) == 0;
  const int64_t n4 = vec ? n >> 2 : 0;
  for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < n4; q += stride) {
    const int64_t i = q << 2;
    float p[4], g[4], m[4], v[4];
    const float4 g4 = *reinterpret_cast<const float4*>(grad + i);
    const float4 m4 = *reinterpret_cast<const float4*>(exp_avg + i);
    const float4 v4 = *reinterpret_cast<const float4*>(exp_avg_sq + i);
    g[0] = g4.x * grad_scale; g[1] = g4.y * grad_scale; g[2] = g4.z * grad_scale; g[3] = g4.w * grad_scale;
    m[0] = m4.x; m[1] = m4.y; m[2] = m4.z; m[3] = m4.w;
    v[0] = v4.x; v[1] = v4.y; v[2] = v4.z; v[3] = v4.w;
    if (master != nullptr) {
      const float4 p4 = *reinterpret_cast<const float4*>(master + i);
      p[0] = p4.x; p[1] = p4.y; p[2] = p4.z; p[3] = p4.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) p[j] = pd_to_float(w_read[i + j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) adam_update(p[j], g[j], m[j], v[j], beta1, beta2, eps, wd, step_size, bias_c2_sqrt);
    *reinterpret_cast<float4*>(exp_avg + i) = make_float4(m[0], m[1], m[2], m[3]);
    *reinterpret_cast<float4*>(exp_avg_sq + i) = make_float4(v[0], v[1], v[2], v[3]);
    if (master != nullptr) *reinterpret_cast<float4*>(master + i) = make_float4(p[0], p[1], p[2], p[3]);
    store4(w_write + i, p);
  }
  // tail, or everything when the pointers are not aligned
  for (int64_t i = (n4 << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float p = master ? master[i] : pd_to_float(w_read[i]);
    float m = exp_avg[i], v = exp_avg_sq[i];
    adam_update(p, grad[i] * grad_scale, m, v, beta1, beta2, eps, wd, step_size, bias_c2_sqrt);
    exp_avg[i] = m;
    exp_avg_sq[i] = v;
    if (master) master[i] = p;
    w_write[i] = pd_from_float<WT>(p);
  }
}

template <typename T>
__global__ void __launch_bounds__(kOptThreads)
scale_kernel(T* __restrict__ x, int64_t n, float s) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) x[i] = pd_from_float<T>(pd_to_float(x[i]) * s);
}

template <typename D, typename S>
__global__ void __launch_bounds__(kOptThreads)
convert_kernel(D* __restrict__ dst, const S* __restrict__ src, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = pd_from_float<D>(pd_to_float(src[i]));
}

int grid_for(int64_t work_items) {
  int64_t blocks = (work_items + kOptThreads - 1) / kOptThreads;
  int64_t cap = (int64_t)pd_num_sms() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace

// See include/pipedream_b200.h for the argument contract.
PD_EXPORT int pd_opt_sgd_multi_tensor(void* arena, int64_t slot_stride, int read_slot,
                                      int write_slot, int w_dtype, float* master,
                                      const float* grad, float* momentum_buf, int64_t n,
                                      float lr, float momentum, float dampening,
                                      float weight_decay, int nesterov, int first_step,
                                      float grad_scale, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(arena && grad && n >= 0, "pd_opt_sgd_multi_tensor: null arena/grad or n<0");
  PD_REQUIRE(read_slot >= 0 && write_slot >= 0 && slot_stride >= n,
             "pd_opt_sgd_multi_tensor: bad slot arguments");
  PD_REQUIRE(momentum == 0.f || momentum_buf, "pd_opt_sgd_multi_tensor: momentum needs a buffer");
  PD_REQUIRE(w_dtype == PD_F32 || w_dtype == PD_BF16, "pd_opt_sgd_multi_tensor: bad dtype");
  PD_REQUIRE(w_dtype == PD_F32 || master, "pd_opt_sgd_multi_tensor: bf16 weights need an fp32 master");
  PD_REQUIRE((slot_stride % 8) == 0, "pd_opt_sgd_multi_tensor: slot stride must be a multiple of 8 elements");
  if (n == 0) return PD_OK;
  cudaStream_t s = (cudaStream_t)stream;
  int grid = grid_for((n + 3) / 4);
  if (w_dtype == PD_F32) {
    float* base = (float*)arena;
    sgd_ring_kernel<float><<<grid, kOptThreads, 0, s>>>(
        base + (int64_t)read_slot * slot_stride, base + (int64_t)write_slot * slot_stride, master,
        grad, momentum_buf, n, lr, momentum, dampening, weight_decay, nesterov, first_step,
        grad_scale);
  } else {
    __nv_bfloat16* base = (__nv_bfloat16*)arena;
    sgd_ring_kernel<__nv_bfloat16><<<grid, kOptThreads, 0, s>>>(
        base + (int64_t)read_slot * slot_stride, base + (int64_t)write_slot * slot_stride, master,
        grad, momentum_buf, n, lr, momentum, dampening, weight_decay, nesterov, first_step,
        grad_scale);
  }
  PD_LAUNCH_CHECK("sgd_ring_kernel");
  return PD_OK;
}

PD_EXPORT int pd_opt_adam_multi_tensor(void* arena, int64_t slot_stride, int read_slot,
                                       int write_slot, int w_dtype, float* master,
                                       const float* grad, float* exp_avg, float* exp_avg_sq,
                                       int64_t n, float lr, float beta1, float beta2, float eps,
                                       float weight_decay, int64_t step, float grad_scale,
                                       void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(arena && grad && exp_avg && exp_avg_sq && n >= 0, "pd_opt_adam_multi_tensor: null pointer or n<0");
  PD_REQUIRE(read_slot >= 0 && write_slot >= 0 && slot_stride >= n, "pd_opt_adam_multi_tensor: bad slot arguments");
  PD_REQUIRE(step >= 1, "pd_opt_adam_multi_tensor: step counts from 1");
  PD_REQUIRE(w_dtype == PD_F32 || w_dtype == PD_BF16, "pd_opt_adam_multi_tensor: bad dtype");
  PD_REQUIRE(w_dtype == PD_F32 || master, "pd_opt_adam_multi_tensor: bf16 weights need an fp32 master");
  if (n == 0) return PD_OK;
  cudaStream_t s = (cudaStream_t)stream;
  // Bias corrections in double on the host, as torch.optim.Adam does in Python floats.
  double bc1 = 1.0 - pow((double)beta1, (double)step);
  double bc2 = 1.0 - pow((double)beta2, (double)step);
  float bias_c1 = (float)bc1;
  float bias_c2_sqrt = (float)sqrt(bc2);
  int grid = grid_for(n);
  if (w_dtype == PD_F32) {
    float* base = (float*)arena;
    adam_ring_kernel<float><<<grid, kOptThreads, 0, s>>>(
        base + (int64_t)read_slot * slot_stride, base + (int64_t)write_slot * slot_stride, master,
        grad, exp_avg, exp_avg_sq, n, lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2_sqrt,
        grad_scale);
  } else {
    __nv_bfloat16* base = (__nv_bfloat16*)arena;
    adam_ring_kernel<__nv_bfloat16><<<grid, kOptThreads, 0, s>>>(
        base + (int64_t)read_slot * slot_stride, base + (int64_t)write_slot * slot_stride, master,
        grad, exp_avg, exp_avg_sq, n, lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2_sqrt,
        grad_scale);
  }
  PD_LAUNCH_CHECK("adam_ring_kernel");
  return PD_OK;
}

PD_EXPORT int pd_scale(void* x, int64_t n, int dtype, float s, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x && n >= 0, "pd_scale: null pointer or n<0");
  if (n == 0) return PD_OK;
  if (dtype == PD_F32)
    scale_kernel<float><<<grid_for(n), kOptThreads, 0, (cudaStream_t)stream>>>((float*)x, n, s);
  else if (dtype == PD_BF16)
    scale_kernel<__nv_bfloat16><<<grid_for(n), kOptThreads, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, n, s);
  else PD_REQUIRE(false, "pd_scale: bad dtype");
  PD_LAUNCH_CHECK("scale_kernel");
  return PD_OK;
}

PD_EXPORT int pd_convert(void* dst, int dst_dtype, const void* src, int src_dtype, int64_t n,
                         void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(dst && src && n >= 0, "pd_convert: null pointer or n<0");
  if (n == 0) return PD_OK;
  cudaStream_t s = (cudaStream_t)stream;
  int g = grid_for(n);
  if (dst_dtype == PD_BF16 && src_dtype == PD_F32)
    convert_kernel<__nv_bfloat16, float><<<g, kOptThreads, 0, s>>>((__nv_bfloat16*)dst, (const float*)src, n);
  else if (dst_dtype == PD_F32 && src_dtype == PD_BF16)
    convert_kernel<float, __nv_bfloat16><<<g, kOptThreads, 0, s>>>((float*)dst, (const __nv_bfloat16*)src, n);
  else if (dst_dtype == PD_F32 && src_dtype == PD_F32)
    convert_kernel<float, float><<<g, kOptThreads, 0, s>>>((float*)dst, (const float*)src, n);
  else if (dst_dtype == PD_BF16 && src_dtype == PD_BF16)
    convert_kernel<__nv_bfloat16, __nv_bfloat16><<<g, kOptThreads, 0, s>>>((__nv_bfloat16*)dst, (const __nv_bfloat16*)src, n);
  else PD_REQUIRE(false, "pd_convert: bad dtype");
  PD_LAUNCH_CHECK("convert_kernel");
  return PD_OK;
}
