// Layout kernels for the convolution and pooling variants of the ResNet-50 stages that are not
// 3x3 / stride 1 (runtime/image_classification/models/resnet50/gpus=4/stage0.py:10-13: 7x7 stride 2,
// 1x1 and 3x3 stride 2, MaxPool2d(3, 2, 1), AvgPool2d(7)).  Those convolutions run as a patch
// matrix (im2col) through the same contraction kernels as everything else; their input gradient is
// gathered back from the patch-matrix gradient (col2im) straight into padded NHWC.
#include "pd_common.cuh"

namespace {

constexpr int kThreads = 256;

int grid_for(int64_t total, int per_sm = 16) {
  int64_t blocks = (total + kThreads - 1) / kThreads;
  int64_t cap = (int64_t)pd_num_sms() * per_sm;
  return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

// dst[(n,ho,wo), (r*kw+s)*C + c] = src[n, c, ho*stride - pad + r, wo*stride - pad + s] (0 outside, 0 for k >= kh*kw*C)
template <typename S, typename D>
__global__ void __launch_bounds__(kThreads)
im2col_kernel(const S* __restrict__ src, int64_t sN, int64_t sC, int64_t sH, int64_t sW, int N, int C, int H, int W,
              int kh, int kw, int stride, int pad, int Ho, int Wo, int Kpad, D* __restrict__ dst) {
  const int64_t total = (int64_t)N * Ho * Wo * Kpad;
  const int K = kh * kw * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int k = (int)(i % Kpad);
    const int64_t p = i / Kpad;
    const int wo = (int)(p % Wo), ho = (int)((p / Wo) % Ho), n = (int)(p / ((int64_t)Wo * Ho));
    float v = 0.f;
    if (k < K) {
      const int t = k / C, c = k - t * C;
      const int h = ho * stride - pad + t / kw, w = wo * stride - pad + t % kw;
      if (h >= 0 && h < H && w >= 0 && w < W) v = pd_to_float(src[n * sN + c * sC + h * sH + w * sW]);
    }
    dst[i] = pd_from_float<D>(v);
  }
}

// dx_pad[n, h+1, w+1, c] = sum over taps (r,s) with (h + pad - r) % stride == 0 etc. of dcol[(n,ho,wo), (r*kw+s)*C + c]
template <typename T>
__global__ void __launch_bounds__(kThreads)
col2im_kernel(const T* __restrict__ dcol, int N, int C, int H, int W, int kh, int kw, int stride, int pad, int Ho, int Wo,
              int Kpad, T* __restrict__ dx) {
  const int Hp = H + 2, Wp = W + 2;
  const int64_t total = (int64_t)N * Hp * Wp * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const int64_t p = i / C;
    const int wp = (int)(p % Wp), hp = (int)((p / Wp) % Hp), n = (int)(p / ((int64_t)Wp * Hp));
    float acc = 0.f;
    if (hp >= 1 && hp <= H && wp >= 1 && wp <= W) {
      const int h = hp - 1, w = wp - 1;
      for (int r = 0; r < kh; ++r) {
        const int hn = h + pad - r;
        if (hn < 0 || hn % stride) continue;
        const int ho = hn / stride;
        if (ho >= Ho) continue;
        for (int s = 0; s < kw; ++s) {
          const int wn = w + pad - s;
          if (wn < 0 || wn % stride) continue;
          const int wo = wn / stride;
          if (wo >= Wo) continue;
          acc += pd_to_float(dcol[(((int64_t)n * Ho + ho) * Wo + wo) * Kpad + (r * kw + s) * C + c]);
        }
      }
    }
    dx[i] = pd_from_float<T>(acc);
  }
}

// MaxPool2d(kernel 3, stride 2, padding 1) on padded NHWC; the padding of the pool counts as -inf.
template <typename T>
__global__ void __launch_bounds__(kThreads)
maxpool3s2_fwd_kernel(const T* __restrict__ x, int N, int C, int H, int W, int Ho, int Wo, T* __restrict__ y,
                      unsigned char* __restrict__ amax) {
  const int Hp = H + 2, Wp = W + 2, Hop = Ho + 2, Wop = Wo + 2;
  const int64_t total = (int64_t)N * Hop * Wop * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const int64_t p = i / C;
    const int wop = (int)(p % Wop), hop = (int)((p / Wop) % Hop), n = (int)(p / ((int64_t)Wop * Hop));
    float m = 0.f;
    if (hop >= 1 && hop <= Ho && wop >= 1 && wop <= Wo) {
      m = -INFINITY;
      int am = 0;
      const int h0 = (hop - 1) * 2 - 1, w0 = (wop - 1) * 2 - 1;
      for (int r = 0; r < 3; ++r)
        for (int s = 0; s < 3; ++s) {
          const int h = h0 + r, w = w0 + s;
          if (h >= 0 && h < H && w >= 0 && w < W) {
            const float v = pd_to_float(x[(((int64_t)n * Hp + h + 1) * Wp + w + 1) * C + c]);
            if (v > m) { m = v; am = r * 3 + s; }
          }
        }
      if (amax != nullptr) amax[(((int64_t)n * Ho + hop - 1) * Wo + wop - 1) * C + c] = (unsigned char)am;
    }
    y[i] = pd_from_float<T>(m);
  }
}

// The gradient of a window goes to its first maximum in (h,w) scan order, as ATen's max_pool2d does; the forward
// recorded that position (r*3+s) per output element.
template <typename T>
__global__ void __launch_bounds__(kThreads)
maxpool3s2_bwd_kernel(const unsigned char* __restrict__ amax, const T* __restrict__ dy, int N, int C, int H, int W, int Ho,
                      int Wo, T* __restrict__ dx) {
  const int Hp = H + 2, Wp = W + 2, Hop = Ho + 2, Wop = Wo + 2;
  const int64_t total = (int64_t)N * Hp * Wp * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const int64_t p = i / C;
    const int wp = (int)(p % Wp), hp = (int)((p / Wp) % Hp), n = (int)(p / ((int64_t)Wp * Hp));
    float g = 0.f;
    if (hp >= 1 && hp <= H && wp >= 1 && wp <= W) {
      const int h = hp - 1, w = wp - 1;
      for (int ho = max(0, h / 2); ho <= min(Ho - 1, (h + 1) / 2); ++ho)
        for (int wo = max(0, w / 2); wo <= min(Wo - 1, (w + 1) / 2); ++wo) {
          const int mine = (h - (ho * 2 - 1)) * 3 + (w - (wo * 2 - 1));
          if (amax[(((int64_t)n * Ho + ho) * Wo + wo) * C + c] == mine)
            g += pd_to_float(dy[(((int64_t)n * Hop + ho + 1) * Wop + wo + 1) * C + c]);
        }
    }
    dx[i] = pd_from_float<T>(g);
  }
}

// Global average pool: y[n, c] = mean over the H*W interior pixels of x_pad[n, :, :, c].
template <typename T>
__global__ void __launch_bounds__(kThreads)
avgpool_fwd_kernel(const T* __restrict__ x, int N, int C, int H, int W, T* __restrict__ y) {
  const int Hp = H + 2, Wp = W + 2;
  const int64_t total = (int64_t)N * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C), n = (int)(i / C);
    float acc = 0.f;
    for (int h = 1; h <= H; ++h)
      for (int w = 1; w <= W; ++w) acc += pd_to_float(x[(((int64_t)n * Hp + h) * Wp + w) * C + c]);
    y[i] = pd_from_float<T>(acc / (float)(H * W));
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
avgpool_bwd_kernel(const T* __restrict__ dy, int N, int C, int H, int W, T* __restrict__ dx) {
  const int Hp = H + 2, Wp = W + 2;
  const int64_t total = (int64_t)N * Hp * Wp * C;
  const float inv = 1.f / (float)(H * W);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const int64_t p = i / C;
    const int wp = (int)(p % Wp), hp = (int)((p / Wp) % Hp), n = (int)(p / ((int64_t)Wp * Hp));
    const bool in = hp >= 1 && hp <= H && wp >= 1 && wp <= W;
    dx[i] = pd_from_float<T>(in ? pd_to_float(dy[(int64_t)n * C + c]) * inv : 0.f);
  }
}


// ------------------------------------------------------------------------------------------------
// 16-byte variants (bf16, channels innermost, C % 8 == 0): one thread per 8 channels
// ------------------------------------------------------------------------------------------------
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

// src: bf16, element strides sN/sH/sW (multiples of 8), channel stride 1.  dst: [rows, Kpad] bf16.
__global__ void __launch_bounds__(kThreads)
im2col_v8_kernel(const __nv_bfloat16* __restrict__ src, int64_t sN, int64_t sH, int64_t sW, int N, int C, int H, int W,
                 int kh, int kw, int stride, int pad, int Ho, int Wo, int Kpad, uint4* __restrict__ dst) {
  const int KV = Kpad / 8;
  const int64_t total = (int64_t)N * Ho * Wo * KV;
  const int K = kh * kw * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int k = (int)(i % KV) * 8;
    const int64_t p = i / KV;
    const int wo = (int)(p % Wo), ho = (int)((p / Wo) % Ho), n = (int)(p / ((int64_t)Wo * Ho));
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (k < K) {
      const int t = k / C, c = k - t * C;
      const int h = ho * stride - pad + t / kw, w = wo * stride - pad + t % kw;
      if (h >= 0 && h < H && w >= 0 && w < W)
        v = *reinterpret_cast<const uint4*>(src + n * sN + h * sH + w * sW + c);
    }
    dst[i] = v;
  }
}

// Any source layout / channel count (the 3-channel fp32 NCHW network input): 8 consecutive patch-matrix
// columns per thread, gathered one by one, stored as one 16-byte vector.
template <typename S>
__global__ void __launch_bounds__(kThreads)
im2col_gather8_kernel(const S* __restrict__ src, int64_t sN, int64_t sC, int64_t sH, int64_t sW, int N, int C, int H, int W,
                      int kh, int kw, int stride, int pad, int Ho, int Wo, int Kpad, uint4* __restrict__ dst) {
  // per patch-matrix column: offset of (c, r, s) inside an image and (r, s) packed; built once per block so
  // that the inner loop has no integer division
  extern __shared__ int tab[];
  const int K = kh * kw * C;
  for (int k = threadIdx.x; k < Kpad; k += kThreads) {
    int off = 0, rs = 0xffff;
    if (k < K) {
      const int t = k / C, c = k - t * C;
      const int r = t / kw, s_ = t - r * kw;
      off = (int)(c * sC + r * sH + s_ * sW);
      rs = (r << 8) | s_;
    }
    tab[2 * k] = off;
    tab[2 * k + 1] = rs;
  }
  __syncthreads();
  const int KV = Kpad / 8;
  const int64_t total = (int64_t)N * Ho * Wo * KV;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int k0 = (int)(i % KV) * 8;
    const int64_t p = i / KV;
    const int wo = (int)(p % Wo), ho = (int)((p / Wo) % Ho), n = (int)(p / ((int64_t)Wo * Ho));
    const int hb = ho * stride - pad, wb = wo * stride - pad;
    const S* base = src + n * sN + hb * sH + wb * sW;
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int off = tab[2 * (k0 + j)], rs = tab[2 * (k0 + j) + 1];
      const int h = hb + (rs >> 8), w = wb + (rs & 0xff);
      f[j] = (rs != 0xffff && h >= 0 && h < H && w >= 0 && w < W) ? pd_to_float(base[off]) : 0.f;
    }
    dst[i] = pack8(f);
  }
}

__global__ void __launch_bounds__(kThreads)
col2im_v8_kernel(const __nv_bfloat16* __restrict__ dcol, int N, int C, int H, int W, int kh, int kw, int stride, int pad,
                 int Ho, int Wo, int Kpad, uint4* __restrict__ dx) {
  const int Hp = H + 2, Wp = W + 2, C8 = C / 8;
  const int64_t total = (int64_t)N * Hp * Wp * C8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C8) * 8;
    const int64_t p = i / C8;
    const int wp = (int)(p % Wp), hp = (int)((p / Wp) % Hp), n = (int)(p / ((int64_t)Wp * Hp));
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    if (hp >= 1 && hp <= H && wp >= 1 && wp <= W) {
      const int h = hp - 1, w = wp - 1;
      for (int r = 0; r < kh; ++r) {
        const int hn = h + pad - r;
        if (hn < 0 || hn % stride) continue;
        const int ho = hn / stride;
        if (ho >= Ho) continue;
        for (int s = 0; s < kw; ++s) {
          const int wn = w + pad - s;
          if (wn < 0 || wn % stride) continue;
          const int wo = wn / stride;
          if (wo >= Wo) continue;
          const uint4 v = *reinterpret_cast<const uint4*>(dcol + (((int64_t)n * Ho + ho) * Wo + wo) * Kpad + (r * kw + s) * C + c);
          float f[8];
          unpack8(v, f);
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] += f[k];
        }
      }
    }
    dx[i] = pack8(acc);
  }
}

__global__ void __launch_bounds__(kThreads)
maxpool3s2_fwd_v8_kernel(const uint4* __restrict__ x, int N, int C8, int H, int W, int Ho, int Wo, uint4* __restrict__ y,
                         uint2* __restrict__ amax) {
  const int Hp = H + 2, Wp = W + 2, Hop = Ho + 2, Wop = Wo + 2;
  const int64_t total = (int64_t)N * Hop * Wop * C8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C8);
    const int64_t p = i / C8;
    const int wop = (int)(p % Wop), hop = (int)((p / Wop) % Hop), n = (int)(p / ((int64_t)Wop * Hop));
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (hop >= 1 && hop <= Ho && wop >= 1 && wop <= Wo) {
      float m[8];
      unsigned int am[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) { m[k] = -INFINITY; am[k] = 0u; }
      const int h0 = (hop - 1) * 2 - 1, w0 = (wop - 1) * 2 - 1;
#pragma unroll
      for (int r = 0; r < 3; ++r)
#pragma unroll
        for (int s = 0; s < 3; ++s) {
          const int h = h0 + r, w = w0 + s;
          if (h >= 0 && h < H && w >= 0 && w < W) {
            float f[8];
            unpack8(x[(((int64_t)n * Hp + h + 1) * Wp + w + 1) * C8 + c], f);
#pragma unroll
            for (int k = 0; k < 8; ++k)
              if (f[k] > m[k]) { m[k] = f[k]; am[k] = (unsigned int)(r * 3 + s); }
          }
        }
      out = pack8(m);
      if (amax != nullptr)
        amax[(((int64_t)n * Ho + hop - 1) * Wo + wop - 1) * C8 + c] =
            make_uint2(am[0] | (am[1] << 8) | (am[2] << 16) | (am[3] << 24), am[4] | (am[5] << 8) | (am[6] << 16) | (am[7] << 24));
    }
    y[i] = out;
  }
}

__global__ void __launch_bounds__(kThreads)
maxpool3s2_bwd_v8_kernel(const uint2* __restrict__ amax, const uint4* __restrict__ dy, int N, int C8, int H, int W, int Ho,
                         int Wo, uint4* __restrict__ dx) {
  const int Hp = H + 2, Wp = W + 2, Hop = Ho + 2, Wop = Wo + 2;
  const int64_t total = (int64_t)N * Hp * Wp * C8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C8);
    const int64_t p = i / C8;
    const int wp = (int)(p % Wp), hp = (int)((p / Wp) % Hp), n = (int)(p / ((int64_t)Wp * Hp));
    float g[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = 0.f;
    if (hp >= 1 && hp <= H && wp >= 1 && wp <= W) {
      const int h = hp - 1, w = wp - 1;
      for (int ho = max(0, h / 2); ho <= min(Ho - 1, (h + 1) / 2); ++ho)
        for (int wo = max(0, w / 2); wo <= min(Wo - 1, (w + 1) / 2); ++wo) {
          const unsigned int mine = (unsigned int)((h - (ho * 2 - 1)) * 3 + (w - (wo * 2 - 1)));
          const uint2 a = amax[(((int64_t)n * Ho + ho) * Wo + wo) * C8 + c];
          float d[8];
          unpack8(dy[(((int64_t)n * Hop + ho + 1) * Wop + wo + 1) * C8 + c], d);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const unsigned int ak = ((k < 4 ? a.x : a.y) >> (8 * (k & 3))) & 0xffu;
            if (ak == mine) g[k] += d[k];
          }
        }
    }
    dx[i] = pack8(g);
  }
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

#define PD_T2(dtype, ...)                                               \
  if (dtype == PD_F32) { using T = float; __VA_ARGS__ }                 \
  else if (dtype == PD_BF16) { using T = __nv_bfloat16; __VA_ARGS__ }   \
  else { pd_set_error("bad dtype %d", dtype); return PD_ERR_INVALID; }

PD_EXPORT int pd_im2col(const void* src, int src_dtype, int64_t sN, int64_t sC, int64_t sH, int64_t sW, int N, int C,
                        int H, int W, int kh, int kw, int stride, int pad, int Ho, int Wo, int Kpad, void* dst,
                        int dst_dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(src && dst && N > 0 && C > 0 && H > 0 && W > 0 && kh > 0 && kw > 0 && stride > 0 && pad >= 0 && Ho > 0 && Wo > 0 &&
             Kpad >= kh * kw * C, "pd_im2col: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t total = (int64_t)N * Ho * Wo * Kpad;
  const int grid = grid_for(total);
  if (src_dtype == PD_BF16 && dst_dtype == PD_BF16 && sC == 1 && (C % 8) == 0 && (Kpad % 8) == 0 && (sN % 8) == 0 &&
      (sH % 8) == 0 && (sW % 8) == 0 && aligned16(src) && aligned16(dst)) {
    im2col_v8_kernel<<<grid_for(total / 8), kThreads, 0, s>>>((const __nv_bfloat16*)src, sN, sH, sW, N, C, H, W, kh, kw, stride, pad,
                                                              Ho, Wo, Kpad, (uint4*)dst);
  } else if (dst_dtype == PD_BF16 && (Kpad % 8) == 0 && Kpad <= 4096 && kh < 255 && kw < 255 && aligned16(dst) &&
             (int64_t)C * sC + (int64_t)kh * sH + (int64_t)kw * sW < (1ll << 31)) {
    if (src_dtype == PD_F32)
      im2col_gather8_kernel<float><<<grid_for(total / 8), kThreads, (size_t)Kpad * 8, s>>>((const float*)src, sN, sC, sH, sW, N, C, H, W, kh, kw,
                                                                            stride, pad, Ho, Wo, Kpad, (uint4*)dst);
    else if (src_dtype == PD_BF16)
      im2col_gather8_kernel<__nv_bfloat16><<<grid_for(total / 8), kThreads, (size_t)Kpad * 8, s>>>((const __nv_bfloat16*)src, sN, sC, sH, sW, N, C, H,
                                                                                    W, kh, kw, stride, pad, Ho, Wo, Kpad, (uint4*)dst);
    else PD_REQUIRE(false, "pd_im2col: bad dtype combination");
  } else if (src_dtype == PD_F32 && dst_dtype == PD_F32)
    im2col_kernel<float, float><<<grid, kThreads, 0, s>>>((const float*)src, sN, sC, sH, sW, N, C, H, W, kh, kw, stride, pad, Ho, Wo, Kpad, (float*)dst);
  else if (src_dtype == PD_F32 && dst_dtype == PD_BF16)
    im2col_kernel<float, __nv_bfloat16><<<grid, kThreads, 0, s>>>((const float*)src, sN, sC, sH, sW, N, C, H, W, kh, kw, stride, pad, Ho, Wo, Kpad, (__nv_bfloat16*)dst);
  else if (src_dtype == PD_BF16 && dst_dtype == PD_BF16)
    im2col_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)src, sN, sC, sH, sW, N, C, H, W, kh, kw, stride, pad, Ho, Wo, Kpad, (__nv_bfloat16*)dst);
  else PD_REQUIRE(false, "pd_im2col: bad dtype combination");
  PD_LAUNCH_CHECK("im2col_kernel");
  return PD_OK;
}

PD_EXPORT int pd_col2im_pnhwc(const void* dcol, int N, int C, int H, int W, int kh, int kw, int stride, int pad, int Ho,
                              int Wo, int Kpad, void* dx_pad, int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(dcol && dx_pad && N > 0 && C > 0 && H > 0 && W > 0 && kh > 0 && kw > 0 && stride > 0 && Ho > 0 && Wo > 0,
             "pd_col2im_pnhwc: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t total = (int64_t)N * (H + 2) * (W + 2) * C;
  if (dtype == PD_BF16 && (C % 8) == 0 && (Kpad % 8) == 0 && aligned16(dcol) && aligned16(dx_pad)) {
    col2im_v8_kernel<<<grid_for(total / 8), kThreads, 0, s>>>((const __nv_bfloat16*)dcol, N, C, H, W, kh, kw, stride, pad, Ho, Wo, Kpad,
                                                              (uint4*)dx_pad);
  } else {
    PD_T2(dtype, col2im_kernel<T><<<grid_for(total), kThreads, 0, s>>>((const T*)dcol, N, C, H, W, kh, kw, stride, pad, Ho, Wo, Kpad, (T*)dx_pad);)
  }
  PD_LAUNCH_CHECK("col2im_kernel");
  return PD_OK;
}

PD_EXPORT int pd_maxpool3s2_fwd(const void* x_pad, int N, int C, int H, int W, void* y_pad, unsigned char* argmax, int dtype,
                                void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x_pad && y_pad && N > 0 && C > 0 && H > 0 && W > 0, "pd_maxpool3s2_fwd: bad arguments");
  const int Ho = (H + 2 - 3) / 2 + 1, Wo = (W + 2 - 3) / 2 + 1;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t total = (int64_t)N * (Ho + 2) * (Wo + 2) * C;
  if (dtype == PD_BF16 && (C % 8) == 0 && aligned16(x_pad) && aligned16(y_pad) && (((uintptr_t)argmax) & 7) == 0) {
    maxpool3s2_fwd_v8_kernel<<<grid_for(total / 8), kThreads, 0, s>>>((const uint4*)x_pad, N, C / 8, H, W, Ho, Wo, (uint4*)y_pad,
                                                                      (uint2*)argmax);
  } else {
    PD_T2(dtype, maxpool3s2_fwd_kernel<T><<<grid_for(total), kThreads, 0, s>>>((const T*)x_pad, N, C, H, W, Ho, Wo, (T*)y_pad, argmax);)
  }
  PD_LAUNCH_CHECK("maxpool3s2_fwd_kernel");
  return PD_OK;
}

PD_EXPORT int pd_maxpool3s2_bwd(const unsigned char* argmax, const void* dy_pad, int N, int C, int H, int W, void* dx_pad,
                                int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(argmax && dy_pad && dx_pad && N > 0 && C > 0 && H > 0 && W > 0, "pd_maxpool3s2_bwd: bad arguments");
  const int Ho = (H + 2 - 3) / 2 + 1, Wo = (W + 2 - 3) / 2 + 1;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t total = (int64_t)N * (H + 2) * (W + 2) * C;
  if (dtype == PD_BF16 && (C % 8) == 0 && (((uintptr_t)argmax) & 7) == 0 && aligned16(dy_pad) && aligned16(dx_pad)) {
    maxpool3s2_bwd_v8_kernel<<<grid_for(total / 8), kThreads, 0, s>>>((const uint2*)argmax, (const uint4*)dy_pad, N, C / 8, H, W, Ho,
                                                                      Wo, (uint4*)dx_pad);
  } else {
    PD_T2(dtype, maxpool3s2_bwd_kernel<T><<<grid_for(total), kThreads, 0, s>>>(argmax, (const T*)dy_pad, N, C, H, W, Ho, Wo, (T*)dx_pad);)
  }
  PD_LAUNCH_CHECK("maxpool3s2_bwd_kernel");
  return PD_OK;
}

PD_EXPORT int pd_avgpool_fwd(const void* x_pad, int N, int C, int H, int W, void* y, int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x_pad && y && N > 0 && C > 0 && H > 0 && W > 0, "pd_avgpool_fwd: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  PD_T2(dtype, avgpool_fwd_kernel<T><<<grid_for((int64_t)N * C), kThreads, 0, s>>>((const T*)x_pad, N, C, H, W, (T*)y);)
  PD_LAUNCH_CHECK("avgpool_fwd_kernel");
  return PD_OK;
}

PD_EXPORT int pd_avgpool_bwd(const void* dy, int N, int C, int H, int W, void* dx_pad, int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(dy && dx_pad && N > 0 && C > 0 && H > 0 && W > 0, "pd_avgpool_bwd: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t total = (int64_t)N * (H + 2) * (W + 2) * C;
  PD_T2(dtype, avgpool_bwd_kernel<T><<<grid_for(total), kThreads, 0, s>>>((const T*)dy, N, C, H, W, (T*)dx_pad);)
  PD_LAUNCH_CHECK("avgpool_bwd_kernel");
  return PD_OK;
}
