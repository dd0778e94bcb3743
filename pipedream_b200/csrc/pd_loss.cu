// Criterion kernels: softmax cross-entropy (torch.nn.CrossEntropyLoss, mean
// reduction) and label-smoothed NLL (runtime/translation/seq2seq/train/smoothing.py:23-34).
// Row statistics are accumulated in fp32 whatever the logits dtype.
#include "pd_common.cuh"
#include <mutex>

namespace {

constexpr int kThreads = 256;

// Scratch of pd_softmax_ce_fwd_static: one per-row loss term per logits row.  It is part of the
// library image, so every GPU that loads the library holds these 256 KiB until the process exits.
constexpr int kStaticRowsMax = 65536;
static __device__ __align__(256) float g_static_row_loss[kStaticRowsMax];

__device__ __forceinline__ float block_max(float v, float* sm) {
  v = pd_warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sm[w] = v;
  __syncthreads();
  float r = (threadIdx.x < (blockDim.x >> 5)) ? sm[threadIdx.x] : -INFINITY;
  if (w == 0) { r = pd_warp_max(r); if (l == 0) sm[0] = r; }
  __syncthreads();
  r = sm[0];
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_sum(float v, float* sm) {
  v = pd_warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sm[w] = v;
  __syncthreads();
  float r = (threadIdx.x < (blockDim.x >> 5)) ? sm[threadIdx.x] : 0.f;
  if (w == 0) { r = pd_warp_sum(r); if (l == 0) sm[0] = r; }
  __syncthreads();
  r = sm[0];
  __syncthreads();
  return r;
}

// One block per row.  row_loss[r] = per-row loss term (already weighted),
// lse[r] = log-sum-exp of the row (kept for the backward pass).
//   smoothing == 0, ignore < 0  : plain cross-entropy, row_loss = lse - x[target]
//   label smoothing             : conf*(lse - x[t]) + smoothing*(lse - mean(x)), 0 for rows whose
//                                 target equals padding_idx
template <typename T>
__global__ void __launch_bounds__(kThreads)
softmax_ce_rows_kernel(const T* __restrict__ logits, const int64_t* __restrict__ target, int C,
                       float smoothing, int64_t padding_idx, float* __restrict__ row_loss,
                       float* __restrict__ lse_out) {
  __shared__ float sm[32];
  const int64_t r = blockIdx.x;
  const T* x = logits + r * C;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < C; c += blockDim.x) mx = fmaxf(mx, pd_to_float(x[c]));
  mx = block_max(mx, sm);
  float se = 0.f, sx = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = pd_to_float(x[c]);
    se += __expf(v - mx);
    sx += v;
  }
  se = block_sum(se, sm);
  sx = block_sum(sx, sm);
  if (threadIdx.x == 0) {
    const float lse = mx + logf(se);
    lse_out[r] = lse;
    const int64_t t = target[r];
    float loss = 0.f;
    if (t >= 0 && t < C && !(padding_idx >= 0 && t == padding_idx)) {
      const float nll = lse - pd_to_float(x[t]);
      const float smooth = lse - sx / (float)C;
      loss = (1.f - smoothing) * nll + smoothing * smooth;
    }
    row_loss[r] = loss;
  }
}

// bf16 rows whose length is a multiple of 8 and whose base is 16-byte aligned: one pass over the row with 16-byte
// loads and an online log-sum-exp (running maximum m and sum of exp(x - m) per thread, merged across the block), so
// the logits are read from HBM exactly once.  Same outputs as softmax_ce_rows_kernel.
__global__ void __launch_bounds__(kThreads)
softmax_ce_rows_bf16x8_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ target, int C,
                              float smoothing, int64_t padding_idx, float* __restrict__ row_loss,
                              float* __restrict__ lse_out) {
  __shared__ float sm[32];
  const int64_t r = blockIdx.x;
  const __nv_bfloat16* x = logits + r * C;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const int nv = C >> 3;
  float m = -INFINITY, se = 0.f, sx = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const uint4 pk = __ldg(xv + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
    float v[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      v[2 * e] = f.x; v[2 * e + 1] = f.y;
    }
    float vm = v[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) vm = fmaxf(vm, v[e]);
    const float mn = fmaxf(m, vm);
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) { acc += __expf(v[e] - mn); sx += v[e]; }
    se = se * __expf(m - mn) + acc;          // (m = -inf on the first vector: exp(-inf) = 0)
    m = mn;
  }
  const float mx = block_max(m, sm);
  se = block_sum(m == -INFINITY ? 0.f : se * __expf(m - mx), sm);
  sx = block_sum(sx, sm);
  if (threadIdx.x == 0) {
    const float lse = mx + logf(se);
    lse_out[r] = lse;
    const int64_t t = target[r];
    float loss = 0.f;
    if (t >= 0 && t < C && !(padding_idx >= 0 && t == padding_idx)) {
      const float nll = lse - __bfloat162float(x[t]);
      const float smooth = lse - sx / (float)C;
      loss = (1.f - smoothing) * nll + smoothing * smooth;
    }
    row_loss[r] = loss;
  }
}

// The matching backward pass: 16-byte loads and stores.
__global__ void __launch_bounds__(kThreads)
softmax_ce_bwd_bf16x8_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ target,
                             const float* __restrict__ lse, int C, float smoothing, int64_t padding_idx,
                             const float* __restrict__ upstream, float gscale, __nv_bfloat16* __restrict__ dlogits) {
  const int64_t r = blockIdx.x;
  const uint4* xv = reinterpret_cast<const uint4*>(logits + r * C);
  uint4* dv = reinterpret_cast<uint4*>(dlogits + r * C);
  const int64_t t = target[r];
  const bool dead = !(t >= 0 && t < C) || (padding_idx >= 0 && t == padding_idx);
  const float g = gscale * (upstream ? *upstream : 1.f);
  const float l = lse[r];
  const float conf = 1.f - smoothing, sm_c = smoothing / (float)C;
  const int nv = C >> 3;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (!dead) {
      const uint4 pk = __ldg(xv + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
      __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
      const int c0 = i << 3;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        const float a = g * (__expf(f.x - l) - ((int64_t)(c0 + 2 * e) == t ? conf : 0.f) - sm_c);
        const float b = g * (__expf(f.y - l) - ((int64_t)(c0 + 2 * e + 1) == t ? conf : 0.f) - sm_c);
        o[e] = __floats2bfloat162_rn(a, b);
      }
    }
    dv[i] = out;
  }
}

template <typename T>
void launch_rows(const void* logits, const int64_t* target, int64_t rows, int C, float smoothing, int64_t padding_idx,
                 float* row_loss, float* lse, cudaStream_t s);
template <>
void launch_rows<float>(const void* logits, const int64_t* target, int64_t rows, int C, float smoothing,
                        int64_t padding_idx, float* row_loss, float* lse, cudaStream_t s) {
  softmax_ce_rows_kernel<float><<<(unsigned)rows, kThreads, 0, s>>>((const float*)logits, target, C, smoothing, padding_idx,
                                                                     row_loss, lse);
}
template <>
void launch_rows<__nv_bfloat16>(const void* logits, const int64_t* target, int64_t rows, int C, float smoothing,
                                int64_t padding_idx, float* row_loss, float* lse, cudaStream_t s) {
  if ((C & 7) == 0 && (((uintptr_t)logits) & 15) == 0)
    softmax_ce_rows_bf16x8_kernel<<<(unsigned)rows, kThreads, 0, s>>>((const __nv_bfloat16*)logits, target, C, smoothing,
                                                                       padding_idx, row_loss, lse);
  else
    softmax_ce_rows_kernel<__nv_bfloat16><<<(unsigned)rows, kThreads, 0, s>>>((const __nv_bfloat16*)logits, target, C, smoothing,
                                                                               padding_idx, row_loss, lse);
}

// Deterministic single-block reduction: loss = scale * sum(row_loss).
__global__ void __launch_bounds__(1024)
loss_reduce_kernel(const float* __restrict__ row_loss, int64_t rows, float scale, float* __restrict__ loss) {
  __shared__ float sm[32];
  float acc = 0.f;
  for (int64_t i = threadIdx.x; i < rows; i += blockDim.x) acc += row_loss[i];
  acc = block_sum(acc, sm);
  if (threadIdx.x == 0) *loss = acc * scale;
}

// dlogits[r,c] = gscale * upstream * (conf*(p - onehot) + smoothing*(p - 1/C)), zero for padded rows.
template <typename T>
__global__ void __launch_bounds__(kThreads)
softmax_ce_bwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ target,
                      const float* __restrict__ lse, int C, float smoothing, int64_t padding_idx,
                      const float* __restrict__ upstream, float gscale, T* __restrict__ dlogits) {
  const int64_t r = blockIdx.x;
  const T* x = logits + r * C;
  T* dx = dlogits + r * C;
  const int64_t t = target[r];
  const bool dead = !(t >= 0 && t < C) || (padding_idx >= 0 && t == padding_idx);
  const float g = gscale * (upstream ? *upstream : 1.f);
  const float l = lse[r];
  const float conf = 1.f - smoothing, sm_c = smoothing / (float)C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float v = 0.f;
    if (!dead) {
      const float p = __expf(pd_to_float(x[c]) - l);
      v = g * (p - (c == t ? conf : 0.f) - sm_c);
    }
    dx[c] = pd_from_float<T>(v);
  }
}

}  // namespace

PD_EXPORT int pd_softmax_ce_fwd(const void* logits, int dtype, const int64_t* target, int64_t rows,
                                int C, float smoothing, int64_t padding_idx, float scale,
                                float* row_loss, float* lse, float* loss, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(logits && target && row_loss && lse && loss && rows > 0 && C > 0,
             "pd_softmax_ce_fwd: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PD_F32) launch_rows<float>(logits, target, rows, C, smoothing, padding_idx, row_loss, lse, s);
  else if (dtype == PD_BF16) launch_rows<__nv_bfloat16>(logits, target, rows, C, smoothing, padding_idx, row_loss, lse, s);
  else PD_REQUIRE(false, "pd_softmax_ce_fwd: bad dtype");
  PD_LAUNCH_CHECK("softmax_ce_rows_kernel");
  loss_reduce_kernel<<<1, 1024, 0, s>>>(row_loss, rows, scale, loss);
  PD_LAUNCH_CHECK("loss_reduce_kernel");
  return PD_OK;
}

PD_EXPORT int pd_softmax_ce_bwd(const void* logits, int dtype, const int64_t* target,
                                const float* lse, int64_t rows, int C, float smoothing,
                                int64_t padding_idx, const float* upstream, float gscale,
                                void* dlogits, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(logits && target && lse && dlogits && rows > 0 && C > 0, "pd_softmax_ce_bwd: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PD_F32)
    softmax_ce_bwd_kernel<float><<<(unsigned)rows, kThreads, 0, s>>>((const float*)logits, target, lse, C, smoothing, padding_idx, upstream, gscale, (float*)dlogits);
  else if (dtype == PD_BF16 && (C & 7) == 0 && ((((uintptr_t)logits) | ((uintptr_t)dlogits)) & 15) == 0)
    softmax_ce_bwd_bf16x8_kernel<<<(unsigned)rows, kThreads, 0, s>>>((const __nv_bfloat16*)logits, target, lse, C, smoothing, padding_idx, upstream, gscale, (__nv_bfloat16*)dlogits);
  else if (dtype == PD_BF16)
    softmax_ce_bwd_kernel<__nv_bfloat16><<<(unsigned)rows, kThreads, 0, s>>>((const __nv_bfloat16*)logits, target, lse, C, smoothing, padding_idx, upstream, gscale, (__nv_bfloat16*)dlogits);
  else PD_REQUIRE(false, "pd_softmax_ce_bwd: bad dtype");
  PD_LAUNCH_CHECK("softmax_ce_bwd_kernel");
  return PD_OK;
}


namespace {
std::mutex g_static_mu;
float* g_static_row_loss_addr[64];     // device address of g_static_row_loss, per device ordinal

// In host code `g_static_row_loss` is only a handle for the symbol, not an address a kernel can
// use; the device address is looked up once per device, with that device current.
int static_row_loss_ptr(float** out) {
  int dev = 0;
  PD_CUDA(cudaGetDevice(&dev));
  PD_REQUIRE(dev >= 0 && dev < 64, "pd_softmax_ce_fwd_static: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_static_row_loss_addr[dev] == nullptr) {
    float* p = nullptr;
    PD_CUDA(cudaGetSymbolAddress((void**)&p, g_static_row_loss));
    PD_REQUIRE(p != nullptr, "pd_softmax_ce_fwd_static: the scratch symbol has no device address");
    g_static_row_loss_addr[dev] = p;
  }
  *out = g_static_row_loss_addr[dev];
  return PD_OK;
}
}  // namespace

// Same result as pd_softmax_ce_fwd (loss and lse), but the per-row scratch is a fixed array inside
// the library instead of a caller buffer, and the call makes no device allocation of any kind.
// For hosts that must not allocate once training runs: a stage whose HBM was planned and handed
// out up front (weight-version ring, activation stash), or an embedding runtime that forbids
// cudaMalloc after start-up because it synchronises the device and can fail late.
//   - rows above pd_softmax_ce_static_max_rows() (65536) are rejected with PD_ERR_INVALID;
//   - the first call on each device looks up the array's device address (a host-side runtime
//     query, no allocation); make that first call before starting any stream capture;
//   - all calls on a device share the one array: every call overwrites the rows it uses and reads
//     nothing older, so nothing needs clearing, but two calls that overlap on the GPU (different
//     streams without an ordering between them) race on it.
PD_EXPORT int pd_softmax_ce_fwd_static(const void* logits, int dtype, const int64_t* target, int64_t rows,
                                       int C, float smoothing, int64_t padding_idx, float scale, float* lse,
                                       float* loss, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(logits && target && lse && loss && rows > 0 && C > 0, "pd_softmax_ce_fwd_static: bad arguments");
  PD_REQUIRE(rows <= kStaticRowsMax,
             "pd_softmax_ce_fwd_static: %lld rows exceed the built-in scratch of %d rows; use pd_softmax_ce_fwd "
             "with a caller buffer", (long long)rows, kStaticRowsMax);
  float* row_loss = nullptr;
  rc = static_row_loss_ptr(&row_loss);
  if (rc != PD_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PD_F32) launch_rows<float>(logits, target, rows, C, smoothing, padding_idx, row_loss, lse, s);
  else if (dtype == PD_BF16) launch_rows<__nv_bfloat16>(logits, target, rows, C, smoothing, padding_idx, row_loss, lse, s);
  else PD_REQUIRE(false, "pd_softmax_ce_fwd_static: bad dtype");
  PD_LAUNCH_CHECK("softmax_ce_rows_kernel");
  loss_reduce_kernel<<<1, 1024, 0, s>>>(row_loss, rows, scale, loss);
  PD_LAUNCH_CHECK("loss_reduce_kernel");
  return PD_OK;
}

PD_EXPORT int64_t pd_softmax_ce_static_max_rows() { return kStaticRowsMax; }
