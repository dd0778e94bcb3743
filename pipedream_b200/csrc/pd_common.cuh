// Shared helpers for the pipedream_b200 C-ABI library (sm_100a only).
// Every exported function returns an int status (0 = ok, negative = error) and
// records a thread-local message readable through pd_last_error().
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>

#define PD_OK 0
#define PD_ERR_INVALID (-1)      // bad argument / unsupported shape
#define PD_ERR_CUDA (-2)         // CUDA runtime / launch error
#define PD_ERR_ARCH (-3)         // device is not sm_100
#define PD_ERR_TIMEOUT (-4)      // a bounded device-side wait ran out
#define PD_ERR_STATE (-5)        // object used in the wrong state

#define PD_F32 0
#define PD_BF16 1

#define PD_EXPORT extern "C" __attribute__((visibility("default")))

void pd_set_error(const char* fmt, ...);
int pd_check_device();          // PD_OK when the current device is sm_100
int pd_num_sms();               // SM count of the current device (cached per device)

#define PD_REQUIRE(cond, ...)                          \
  do {                                                 \
    if (!(cond)) {                                     \
      pd_set_error(__VA_ARGS__);                       \
      return PD_ERR_INVALID;                           \
    }                                                  \
  } while (0)

#define PD_CUDA(call)                                                      \
  do {                                                                     \
    cudaError_t e__ = (call);                                              \
    if (e__ != cudaSuccess) {                                              \
      pd_set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), \
                   __FILE__, __LINE__);                                    \
      return PD_ERR_CUDA;                                                  \
    }                                                                      \
  } while (0)

#define PD_LAUNCH_CHECK(name)                                              \
  do {                                                                     \
    cudaError_t e__ = cudaGetLastError();                                  \
    if (e__ != cudaSuccess) {                                              \
      pd_set_error("launch of %s failed: %s", name, cudaGetErrorString(e__)); \
      return PD_ERR_CUDA;                                                  \
    }                                                                      \
  } while (0)

static inline int pd_elem_size(int dtype) { return dtype == PD_BF16 ? 2 : 4; }

// ---- device helpers -------------------------------------------------------
template <typename T> struct PdVec;   // 16-byte vector of T

__device__ __forceinline__ float pd_to_float(float v) { return v; }
__device__ __forceinline__ float pd_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T pd_from_float(float v);
template <> __device__ __forceinline__ float pd_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 pd_from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float pd_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float pd_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
