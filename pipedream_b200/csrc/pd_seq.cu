// Sequence utilities for the translation stages: per-sequence time reversal,
// length masks and the embedding gather / scatter-add.
// Replaces runtime/translation/seq2seq/csrc/pack_utils_kernel.cu:7-63 and
// pack_utils.cpp:13-31; offsets are derived on the device from a device-resident
// lengths vector instead of being built on the host and copied per call.
#include "pd_common.cuh"

namespace {
constexpr int kThreads = 256;

// out[t,b,:] = in[len[b]-1-t, b, :] for t < len[b], else 0.  16-byte vectors when
// the feature size allows; one block per (t,b) row chunk.
template <typename V>
__global__ void __launch_bounds__(kThreads)
revert_varlen_kernel(const V* __restrict__ in, V* __restrict__ out, const int64_t* __restrict__ lengths,
                     int T, int B, int fvec) {
  const int64_t rows = (int64_t)T * B;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int t = (int)(row / B), b = (int)(row % B);
    const int64_t len = lengths[b];
    V* o = out + row * fvec;
    if (t < len) {
      const V* s = in + ((int64_t)(len - 1 - t) * B + b) * fvec;
      for (int i = threadIdx.x; i < fvec; i += blockDim.x) o[i] = s[i];
    } else {
      V z; memset(&z, 0, sizeof(V));
      for (int i = threadIdx.x; i < fvec; i += blockDim.x) o[i] = z;
    }
  }
}

// mask[t,b] = t < len[b]
template <typename T>
__global__ void __launch_bounds__(kThreads)
length_mask_kernel(const int64_t* __restrict__ lengths, int Tn, int B, T* __restrict__ mask, float one) {
  const int64_t total = (int64_t)Tn * B;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / B), b = (int)(i % B);
    mask[i] = (T)(t < lengths[b] ? one : 0.f);
  }
}

// y[r, :] = x[r, :] * mask[r]
template <typename T>
__global__ void __launch_bounds__(kThreads)
mul_rows_kernel(const T* __restrict__ x, const T* __restrict__ mask, T* __restrict__ y, int64_t rows, int F) {
  const int64_t total = rows * F;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    y[i] = pd_from_float<T>(pd_to_float(x[i]) * pd_to_float(mask[i / F]));
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
embedding_fwd_kernel(const int64_t* __restrict__ ids, const T* __restrict__ table, int64_t n, int D,
                     int64_t vocab, T* __restrict__ out) {
  for (int64_t row = blockIdx.x; row < n; row += gridDim.x) {
    int64_t id = ids[row];
    if (id < 0 || id >= vocab) id = 0;
    const T* s = table + id * D;
    T* o = out + row * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = s[i];
  }
}

// dtable[id,:] += dy[row,:] (fp32 accumulate), rows whose id equals padding_idx are skipped.
template <typename T>
__global__ void __launch_bounds__(kThreads)
embedding_bwd_kernel(const int64_t* __restrict__ ids, const T* __restrict__ dy, int64_t n, int D,
                     int64_t vocab, int64_t padding_idx, float* __restrict__ dtable) {
  for (int64_t row = blockIdx.x; row < n; row += gridDim.x) {
    const int64_t id = ids[row];
    if (id < 0 || id >= vocab || id == padding_idx) continue;
    const T* s = dy + row * D;
    float* o = dtable + id * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(o + i, pd_to_float(s[i]));
  }
}
}  // namespace

PD_EXPORT int pd_revert_varlen(const void* in, void* out, const int64_t* lengths, int T, int B,
                               int64_t feature_bytes, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(in && out && lengths && T > 0 && B > 0 && feature_bytes > 0, "pd_revert_varlen: bad arguments");
  PD_REQUIRE(in != out, "pd_revert_varlen: in-place reversal is not supported");
  cudaStream_t s = (cudaStream_t)stream;
  int64_t rows = (int64_t)T * B;
  int grid = (int)(rows < (int64_t)pd_num_sms() * 16 ? rows : (int64_t)pd_num_sms() * 16);
  if (feature_bytes % 16 == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0)
    revert_varlen_kernel<uint4><<<grid, kThreads, 0, s>>>((const uint4*)in, (uint4*)out, lengths, T, B, (int)(feature_bytes / 16));
  else if (feature_bytes % 4 == 0)
    revert_varlen_kernel<uint32_t><<<grid, kThreads, 0, s>>>((const uint32_t*)in, (uint32_t*)out, lengths, T, B, (int)(feature_bytes / 4));
  else if (feature_bytes % 2 == 0)
    revert_varlen_kernel<uint16_t><<<grid, kThreads, 0, s>>>((const uint16_t*)in, (uint16_t*)out, lengths, T, B, (int)(feature_bytes / 2));
  else
    revert_varlen_kernel<uint8_t><<<grid, kThreads, 0, s>>>((const uint8_t*)in, (uint8_t*)out, lengths, T, B, (int)feature_bytes);
  PD_LAUNCH_CHECK("revert_varlen_kernel");
  return PD_OK;
}

// mask_dtype: PD_F32 / PD_BF16, or 2 for uint8 (the reference's set_mask_cpp output type).
PD_EXPORT int pd_length_mask(const int64_t* lengths, int T, int B, void* mask, int mask_dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(lengths && mask && T > 0 && B > 0, "pd_length_mask: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  int64_t total = (int64_t)T * B;
  int grid = (int)((total + kThreads - 1) / kThreads);
  if (mask_dtype == PD_F32) length_mask_kernel<float><<<grid, kThreads, 0, s>>>(lengths, T, B, (float*)mask, 1.f);
  else if (mask_dtype == PD_BF16) length_mask_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(lengths, T, B, (__nv_bfloat16*)mask, 1.f);
  else if (mask_dtype == 2) length_mask_kernel<uint8_t><<<grid, kThreads, 0, s>>>(lengths, T, B, (uint8_t*)mask, 1.f);
  else PD_REQUIRE(false, "pd_length_mask: bad dtype");
  PD_LAUNCH_CHECK("length_mask_kernel");
  return PD_OK;
}

PD_EXPORT int pd_embedding_fwd(const int64_t* ids, const void* table, int64_t n, int D, int64_t vocab,
                               void* out, int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(ids && table && out && n > 0 && D > 0 && vocab > 0, "pd_embedding_fwd: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  int grid = (int)(n < (int64_t)pd_num_sms() * 16 ? n : (int64_t)pd_num_sms() * 16);
  if (dtype == PD_F32) embedding_fwd_kernel<float><<<grid, kThreads, 0, s>>>(ids, (const float*)table, n, D, vocab, (float*)out);
  else if (dtype == PD_BF16) embedding_fwd_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(ids, (const __nv_bfloat16*)table, n, D, vocab, (__nv_bfloat16*)out);
  else PD_REQUIRE(false, "pd_embedding_fwd: bad dtype");
  PD_LAUNCH_CHECK("embedding_fwd_kernel");
  return PD_OK;
}

PD_EXPORT int pd_embedding_bwd(const int64_t* ids, const void* dy, int64_t n, int D, int64_t vocab,
                               int64_t padding_idx, float* dtable, int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(ids && dy && dtable && n > 0 && D > 0 && vocab > 0, "pd_embedding_bwd: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  int grid = (int)(n < (int64_t)pd_num_sms() * 16 ? n : (int64_t)pd_num_sms() * 16);
  if (dtype == PD_F32) embedding_bwd_kernel<float><<<grid, kThreads, 0, s>>>(ids, (const float*)dy, n, D, vocab, padding_idx, dtable);
  else if (dtype == PD_BF16) embedding_bwd_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(ids, (const __nv_bfloat16*)dy, n, D, vocab, padding_idx, dtable);
  else PD_REQUIRE(false, "pd_embedding_bwd: bad dtype");
  PD_LAUNCH_CHECK("embedding_bwd_kernel");
  return PD_OK;
}


// y[r,:] = x[r,:] * mask[r]: the length mask applied to the forward half of the bidirectional encoder
// layer (runtime/translation/seq2seq/models/encoder.py:51,55).
PD_EXPORT int pd_mul_rows(const void* x, const void* mask, void* y, int64_t rows, int F, int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x && mask && y && rows > 0 && F > 0, "pd_mul_rows: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  int64_t blocks = (rows * F + kThreads - 1) / kThreads;
  int grid = (int)(blocks < (int64_t)pd_num_sms() * 16 ? blocks : (int64_t)pd_num_sms() * 16);
  if (dtype == PD_F32) mul_rows_kernel<float><<<grid, kThreads, 0, s>>>((const float*)x, (const float*)mask, (float*)y, rows, F);
  else if (dtype == PD_BF16) mul_rows_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)mask, (__nv_bfloat16*)y, rows, F);
  else PD_REQUIRE(false, "pd_mul_rows: bad dtype");
  PD_LAUNCH_CHECK("mul_rows_kernel");
  return PD_OK;
}
