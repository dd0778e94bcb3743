// Normalised additive (Bahdanau) attention, fused: the reference materialises tanh(q + k + b) as a
// [b, t_q, t_k, n] tensor and runs a dozen pointwise launches around it
// (runtime/translation/seq2seq/models/attention.py:84-170).  Here one kernel per pass keeps that
// tensor in registers:
//   forward : scores = v . tanh(pq + pk + nb), length mask, softmax over t_k, context = probs . keys
//   backward: (1) softmax / context gradients per query row, (2) per (batch, channel) recomputation of
//             tanh for the gradients of pq, pk, v, nb and of the keys.
// pq, pk: projected queries / keys, [b, t_q, n] and [b, t_k, n] contiguous.  keys, context and their
// gradients are addressed with (batch, time) strides so that sequence-first tensors need no copies.
#include "pd_common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxTk = 128;          // keys per sequence the kernels keep in shared memory

template <bool kFast> __device__ __forceinline__ float tanh_(float x) {
  if (kFast) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  }
  return tanhf(x);
}

// grid (t_q, b): one query row per block.
template <typename T, bool kFast>
__global__ void __launch_bounds__(kThreads)
attn_fwd_kernel(const T* __restrict__ pq, const T* __restrict__ pk, const T* __restrict__ keys, int64_t k_sb,
                int64_t k_st, const float* __restrict__ v, const T* __restrict__ nb,
                const int64_t* __restrict__ ctx_len, int tq, int tk, int n, int nk, T* __restrict__ probs,
                T* __restrict__ context, int64_t c_sb, int64_t c_st) {
  extern __shared__ float sm[];            // [n] q + nb, then [kMaxTk] scores
  float* qs = sm;
  float* sc = sm + n;
  const int i = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* q = pq + ((int64_t)b * tq + i) * n;
  for (int c = threadIdx.x; c < n; c += blockDim.x) qs[c] = pd_to_float(q[c]) + pd_to_float(nb[c]);
  __syncthreads();
  for (int j = warp; j < tk; j += kThreads / 32) {
    const T* k = pk + ((int64_t)b * tk + j) * n;
    float acc = 0.f;
    for (int c = lane; c < n; c += 32) acc += v[c] * tanh_<kFast>(qs[c] + pd_to_float(k[c]));
    acc = pd_warp_sum(acc);
    if (lane == 0) sc[j] = (ctx_len != nullptr && j >= ctx_len[b]) ? -65504.f : acc;
  }
  __syncthreads();
  if (warp == 0) {          // softmax over t_k by one warp
    float mx = -INFINITY;
    for (int j = lane; j < tk; j += 32) mx = fmaxf(mx, sc[j]);
    mx = pd_warp_max(mx);
    float se = 0.f;
    for (int j = lane; j < tk; j += 32) { const float e = __expf(sc[j] - mx); sc[j] = e; se += e; }
    se = pd_warp_sum(se);
    const float inv = 1.f / se;
    for (int j = lane; j < tk; j += 32) {
      const float p = sc[j] * inv;
      sc[j] = p;
      probs[((int64_t)b * tq + i) * tk + j] = pd_from_float<T>(p);
    }
  }
  __syncthreads();
  T* ctx = context + b * c_sb + i * c_st;
  for (int c = threadIdx.x; c < nk; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < tk; ++j) acc += sc[j] * pd_to_float(keys[b * k_sb + j * k_st + c]);
    ctx[c] = pd_from_float<T>(acc);
  }
}

// grid (t_q, b): ds[b,i,j] = p_j * (dp_j - sum_j p_j dp_j), dp_j = dcontext[b,i,:] . keys[b,j,:] (+ dprobs).
template <typename T>
__global__ void __launch_bounds__(kThreads)
attn_bwd_softmax_kernel(const T* __restrict__ keys, int64_t k_sb, int64_t k_st, const T* __restrict__ probs,
                        const T* __restrict__ dcontext, int64_t c_sb, int64_t c_st, int tq, int tk, int nk,
                        float* __restrict__ ds) {
  extern __shared__ float sm[];            // [nk] dcontext row, [kMaxTk] dp
  float* dc = sm;
  float* dp = sm + nk;
  const int i = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* g = dcontext + b * c_sb + i * c_st;
  for (int c = threadIdx.x; c < nk; c += blockDim.x) dc[c] = pd_to_float(g[c]);
  __syncthreads();
  for (int j = warp; j < tk; j += kThreads / 32) {
    const T* k = keys + b * k_sb + j * k_st;
    float acc = 0.f;
    for (int c = lane; c < nk; c += 32) acc += dc[c] * pd_to_float(k[c]);
    acc = pd_warp_sum(acc);
    if (lane == 0) dp[j] = acc;
  }
  __syncthreads();
  if (warp == 0) {
    const T* p = probs + ((int64_t)b * tq + i) * tk;
    float dot = 0.f;
    for (int j = lane; j < tk; j += 32) dot += pd_to_float(p[j]) * dp[j];
    dot = pd_warp_sum(dot);
    for (int j = lane; j < tk; j += 32) ds[((int64_t)b * tq + i) * tk + j] = pd_to_float(p[j]) * (dp[j] - dot);
  }
}

// grid (ceil(max(n, nk) / kThreads), b): one channel per thread, all (i, j) pairs of the sequence.
template <typename T, bool kFast>
__global__ void __launch_bounds__(kThreads)
attn_bwd_channels_kernel(const T* __restrict__ pq, const T* __restrict__ pk, const float* __restrict__ v,
                         const T* __restrict__ nb, const T* __restrict__ probs, const float* __restrict__ ds,
                         const T* __restrict__ dcontext, int64_t c_sb, int64_t c_st, int tq, int tk, int n, int nk,
                         T* __restrict__ dpq, T* __restrict__ dpk, T* __restrict__ dkeys, int64_t dk_sb, int64_t dk_st,
                         float* __restrict__ dv, float* __restrict__ dnb) {
  extern __shared__ float sm[];            // [tq*tk] ds, [tq*tk] probs, [tk][kThreads] pk column, [tk][kThreads] dpk
  float* s_ds = sm;
  float* s_p = sm + tq * tk;
  float* s_k = s_p + tq * tk;
  float* s_dk = s_k + tk * kThreads;
  const int b = blockIdx.y;
  const int c = blockIdx.x * kThreads + threadIdx.x;
  for (int e = threadIdx.x; e < tq * tk; e += blockDim.x) {
    s_ds[e] = ds[(int64_t)b * tq * tk + e];
    s_p[e] = pd_to_float(probs[(int64_t)b * tq * tk + e]);
  }
  if (c < n) {
    for (int j = 0; j < tk; ++j) {
      s_k[j * kThreads + threadIdx.x] = pd_to_float(pk[((int64_t)b * tk + j) * n + c]);
      s_dk[j * kThreads + threadIdx.x] = 0.f;
    }
  }
  __syncthreads();
  if (c < n) {
    const float vc = v[c], nbc = pd_to_float(nb[c]);
    float acc_v = 0.f, acc_nb = 0.f;
    for (int i = 0; i < tq; ++i) {
      const float q = pd_to_float(pq[((int64_t)b * tq + i) * n + c]) + nbc;
      float acc_q = 0.f;
      for (int j = 0; j < tk; ++j) {
        const float u = tanh_<kFast>(q + s_k[j * kThreads + threadIdx.x]);
        const float d = s_ds[i * tk + j];
        const float dz = d * vc * (1.f - u * u);
        acc_q += dz;
        s_dk[j * kThreads + threadIdx.x] += dz;
        acc_v += d * u;
      }
      dpq[((int64_t)b * tq + i) * n + c] = pd_from_float<T>(acc_q);
      acc_nb += acc_q;
    }
    for (int j = 0; j < tk; ++j) dpk[((int64_t)b * tk + j) * n + c] = pd_from_float<T>(s_dk[j * kThreads + threadIdx.x]);
    atomicAdd(dv + c, acc_v);
    atomicAdd(dnb + c, acc_nb);
  }
  if (c < nk) {      // gradient of the keys through the weighted sum: dkeys[b,j,c] = sum_i p[b,i,j] dcontext[b,i,c]
    for (int j = 0; j < tk; ++j) {
      float acc = 0.f;
      for (int i = 0; i < tq; ++i) acc += s_p[i * tk + j] * pd_to_float(dcontext[b * c_sb + i * c_st + c]);
      dkeys[b * dk_sb + j * dk_st + c] = pd_from_float<T>(acc);
    }
  }
}

}  // namespace

PD_EXPORT int pd_attn_bahdanau_fwd(int dtype, const void* pq, const void* pk, const void* keys, int64_t k_sb,
                                   int64_t k_st, const float* v, const void* nb, const int64_t* ctx_len, int b,
                                   int tq, int tk, int n, int nk, void* probs, void* context, int64_t c_sb,
                                   int64_t c_st, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(pq && pk && keys && v && nb && probs && context && b > 0 && tq > 0 && tk > 0 && n > 0 && nk > 0,
             "pd_attn_bahdanau_fwd: bad arguments");
  PD_REQUIRE(tk <= kMaxTk, "pd_attn_bahdanau_fwd: at most %d keys per sequence (got %d)", kMaxTk, tk);
  PD_REQUIRE(n <= 8192 && nk <= 8192, "pd_attn_bahdanau_fwd: feature size too large");
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(tq, b);
  const size_t smem = (size_t)(n + kMaxTk) * sizeof(float);
  if (dtype == PD_F32)
    attn_fwd_kernel<float, false><<<grid, kThreads, smem, s>>>((const float*)pq, (const float*)pk, (const float*)keys, k_sb, k_st, v,
                                                               (const float*)nb, ctx_len, tq, tk, n, nk, (float*)probs, (float*)context, c_sb, c_st);
  else if (dtype == PD_BF16)
    attn_fwd_kernel<__nv_bfloat16, true><<<grid, kThreads, smem, s>>>((const __nv_bfloat16*)pq, (const __nv_bfloat16*)pk,
                                                                      (const __nv_bfloat16*)keys, k_sb, k_st, v, (const __nv_bfloat16*)nb,
                                                                      ctx_len, tq, tk, n, nk, (__nv_bfloat16*)probs,
                                                                      (__nv_bfloat16*)context, c_sb, c_st);
  else PD_REQUIRE(false, "pd_attn_bahdanau_fwd: bad dtype");
  PD_LAUNCH_CHECK("attn_fwd_kernel");
  return PD_OK;
}

// dv, dnb: fp32 [n], accumulated into (the caller clears them).  ds_ws: [b, tq, tk] fp32 scratch.
PD_EXPORT int pd_attn_bahdanau_bwd(int dtype, const void* pq, const void* pk, const void* keys, int64_t k_sb,
                                   int64_t k_st, const float* v, const void* nb, const void* probs,
                                   const void* dcontext, int64_t c_sb, int64_t c_st, int b, int tq, int tk, int n,
                                   int nk, void* dpq, void* dpk, void* dkeys, int64_t dk_sb, int64_t dk_st,
                                   float* dv, float* dnb, float* ds_ws, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(pq && pk && keys && v && nb && probs && dcontext && dpq && dpk && dkeys && dv && dnb && ds_ws,
             "pd_attn_bahdanau_bwd: null pointer");
  PD_REQUIRE(b > 0 && tq > 0 && tk > 0 && n > 0 && nk > 0 && tk <= kMaxTk, "pd_attn_bahdanau_bwd: bad sizes");
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem1 = (size_t)(nk + kMaxTk) * sizeof(float);
  const size_t smem2 = ((size_t)2 * tq * tk + (size_t)2 * tk * kThreads) * sizeof(float);
  PD_REQUIRE(smem2 <= 200 * 1024, "pd_attn_bahdanau_bwd: t_q * t_k too large for the shared-memory tile");
  dim3 g1(tq, b);
  const int cmax = n > nk ? n : nk;
  dim3 g2((cmax + kThreads - 1) / kThreads, b);
  if (dtype == PD_F32) {
    attn_bwd_softmax_kernel<float><<<g1, kThreads, smem1, s>>>((const float*)keys, k_sb, k_st, (const float*)probs,
                                                               (const float*)dcontext, c_sb, c_st, tq, tk, nk, ds_ws);
    PD_LAUNCH_CHECK("attn_bwd_softmax_kernel");
    PD_CUDA(cudaFuncSetAttribute(attn_bwd_channels_kernel<float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attn_bwd_channels_kernel<float, false><<<g2, kThreads, smem2, s>>>(
        (const float*)pq, (const float*)pk, v, (const float*)nb, (const float*)probs, ds_ws, (const float*)dcontext, c_sb, c_st,
        tq, tk, n, nk, (float*)dpq, (float*)dpk, (float*)dkeys, dk_sb, dk_st, dv, dnb);
  } else if (dtype == PD_BF16) {
    attn_bwd_softmax_kernel<__nv_bfloat16><<<g1, kThreads, smem1, s>>>((const __nv_bfloat16*)keys, k_sb, k_st,
                                                                       (const __nv_bfloat16*)probs, (const __nv_bfloat16*)dcontext,
                                                                       c_sb, c_st, tq, tk, nk, ds_ws);
    PD_LAUNCH_CHECK("attn_bwd_softmax_kernel");
    PD_CUDA(cudaFuncSetAttribute(attn_bwd_channels_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attn_bwd_channels_kernel<__nv_bfloat16, true><<<g2, kThreads, smem2, s>>>(
        (const __nv_bfloat16*)pq, (const __nv_bfloat16*)pk, v, (const __nv_bfloat16*)nb, (const __nv_bfloat16*)probs, ds_ws,
        (const __nv_bfloat16*)dcontext, c_sb, c_st, tq, tk, n, nk, (__nv_bfloat16*)dpq, (__nv_bfloat16*)dpk,
        (__nv_bfloat16*)dkeys, dk_sb, dk_st, dv, dnb);
  } else {
    PD_REQUIRE(false, "pd_attn_bahdanau_bwd: bad dtype");
  }
  PD_LAUNCH_CHECK("attn_bwd_channels_kernel");
  return PD_OK;
}
