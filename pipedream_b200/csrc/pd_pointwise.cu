// Bandwidth-bound kernels between the contractions of a stage: layout packing,
// ReLU, 2x2 max-pool, dropout, bias-gradient reduction, elementwise add.
//
// Activation layout ("padded NHWC"): a logical [N,C,H,W] tensor is stored as
// [N, H+2, W+2, C] with a one-pixel zero border, channels innermost.  A 3x3
// stride-1 pad-1 convolution then reads tap (r,s) of pixel row p at row
// p + (r-1)*(W+2) + (s-1) of the flattened [N*(H+2)*(W+2), C] matrix, which is
// what lets the implicit-GEMM kernels fetch every tap with a plain 2-D TMA box.
// Every kernel that writes such a buffer keeps the border at zero.
#include <algorithm>

#include "pd_common.cuh"

namespace {

constexpr int kThreads = 256;

inline int grid_cap(int64_t blocks, int per_sm = 8) {
  int64_t cap = (int64_t)pd_num_sms() * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// ---- pack: arbitrary-stride [N,C,H,W] -> padded NHWC ------------------------
template <typename S, typename D>
__global__ void __launch_bounds__(kThreads)
pack_pnhwc_kernel(const S* __restrict__ src, int64_t sN, int64_t sC, int64_t sH, int64_t sW,
                  int N, int C, int H, int W, D* __restrict__ dst) {
  // One block handles one padded row (n, hp); a shared tile transposes [C][W]
  // reads (W fastest for NCHW sources) into [W][C] writes.
  __shared__ float tile[32][33];
  const int Hp = H + 2, Wp = W + 2;
  const int64_t rows = (int64_t)N * Hp;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int n = (int)(row / Hp), hp = (int)(row % Hp);
    D* drow = dst + row * (int64_t)Wp * C;
    if (hp == 0 || hp == Hp - 1) {
      for (int64_t i = threadIdx.x; i < (int64_t)Wp * C; i += blockDim.x) drow[i] = pd_from_float<D>(0.f);
      continue;
    }
    const int h = hp - 1;
    for (int i = threadIdx.x; i < C; i += blockDim.x) {
      drow[i] = pd_from_float<D>(0.f);
      drow[(int64_t)(Wp - 1) * C + i] = pd_from_float<D>(0.f);
    }
    const S* sbase = src + n * sN + h * sH;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (int c0 = 0; c0 < C; c0 += 32) {
      for (int w0 = 0; w0 < W; w0 += 32) {
        __syncthreads();
        if (sC == 1) {  // channels-last source: read along C
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            int w = w0 + ty + j, c = c0 + tx;
            tile[tx][ty + j] = (w < W && c < C) ? pd_to_float(sbase[c * sC + w * sW]) : 0.f;
          }
        } else {        // read along W
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            int c = c0 + ty + j, w = w0 + tx;
            tile[ty + j][tx] = (w < W && c < C) ? pd_to_float(sbase[c * sC + w * sW]) : 0.f;
          }
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          int w = w0 + ty + j, c = c0 + tx;
          if (w < W && c < C) drow[(int64_t)(w + 1) * C + c] = pd_from_float<D>(tile[tx][ty + j]);
        }
      }
    }
  }
}

// ---- unpack: padded NHWC -> contiguous NCHW ---------------------------------
template <typename S, typename D>
__global__ void __launch_bounds__(kThreads)
unpack_pnhwc_kernel(const S* __restrict__ src, int N, int C, int H, int W, D* __restrict__ dst) {
  __shared__ float tile[32][33];
  const int Hp = H + 2, Wp = W + 2;
  const int64_t rows = (int64_t)N * H;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int n = (int)(row / H), h = (int)(row % H);
    const S* srow = src + ((int64_t)(n * Hp + h + 1) * Wp + 1) * C;
    D* dbase = dst + (int64_t)n * C * H * W + (int64_t)h * W;
    for (int c0 = 0; c0 < C; c0 += 32) {
      for (int w0 = 0; w0 < W; w0 += 32) {
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          int w = w0 + ty + j, c = c0 + tx;
          tile[ty + j][tx] = (w < W && c < C) ? pd_to_float(srow[(int64_t)w * C + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          int c = c0 + ty + j, w = w0 + tx;
          if (w < W && c < C) dbase[(int64_t)c * H * W + w] = pd_from_float<D>(tile[tx][ty + j]);
        }
      }
    }
  }
}

// ---- im2col for the 3-channel first convolution -----------------------------
// A[p, k] over padded pixel rows p (border rows all zero), k = (r*3+s)*C + c for
// k < 9*C, zero up to Kpad.  Source is any-stride [N,C,H,W].
template <typename S, typename D>
__global__ void __launch_bounds__(kThreads)
im2col3x3_kernel(const S* __restrict__ src, int64_t sN, int64_t sC, int64_t sH, int64_t sW,
                 int N, int C, int H, int W, int Kpad, D* __restrict__ dst) {
  const int Hp = H + 2, Wp = W + 2;
  const int64_t total = (int64_t)N * Hp * Wp * Kpad;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int k = (int)(i % Kpad);
    const int64_t p = i / Kpad;
    const int wp = (int)(p % Wp);
    const int hp = (int)((p / Wp) % Hp);
    const int n = (int)(p / ((int64_t)Wp * Hp));
    float v = 0.f;
    if (k < 9 * C && hp >= 1 && hp <= H && wp >= 1 && wp <= W) {
      const int t = k / C, c = k % C;
      const int h = hp - 1 + t / 3 - 1, w = wp - 1 + t % 3 - 1;
      if (h >= 0 && h < H && w >= 0 && w < W) v = pd_to_float(src[n * sN + c * sC + h * sH + w * sW]);
    }
    dst[i] = pd_from_float<D>(v);
  }
}

// ---- ReLU --------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
relu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    y[i] = pd_from_float<T>(fmaxf(pd_to_float(x[i]), 0.f));
}

__global__ void __launch_bounds__(kThreads)
relu_fwd_bf16x8_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int64_t n8) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (int64_t)gridDim.x * blockDim.x) {
    uint4 v = x[i];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
    const __nv_bfloat162 z = __float2bfloat162_rn(0.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __hmax2(h[j], z);
    y[i] = v;
  }
}

// dx = dy * (y > 0); y is the ReLU output.
template <typename T>
__global__ void __launch_bounds__(kThreads)
relu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    dx[i] = pd_to_float(y[i]) > 0.f ? dy[i] : pd_from_float<T>(0.f);
}

// Fused: dx = dy * (y > 0) (when y != null) and per-column partial sums of dx
// over a [rows, C] matrix.  partial[block][C] is reduced by colsum_final_kernel.
template <typename T>
__global__ void __launch_bounds__(kThreads)
relu_bwd_colsum_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx,
                       int64_t rows, int C, float* __restrict__ partial) {
  extern __shared__ float sm[];  // [lanes][C]
  const int lanes = kThreads / C > 0 ? kThreads / C : 1;   // C <= kThreads handled per column
  const int cols_per_thread = (C + kThreads - 1) / kThreads;
  // thread -> (lane, col); for C > kThreads each thread walks several columns
  const int lane = (C <= kThreads) ? threadIdx.x / C : 0;
  const int col0 = (C <= kThreads) ? threadIdx.x % C : threadIdx.x;
  const bool active = (C <= kThreads) ? (lane < lanes) : true;
  for (int cc = 0; cc < cols_per_thread; ++cc) {
    const int col = col0 + cc * kThreads;
    float acc = 0.f;
    if (active && col < C) {
      for (int64_t r = (int64_t)blockIdx.x * lanes + lane; r < rows; r += (int64_t)gridDim.x * lanes) {
        const int64_t i = r * C + col;
        float g = pd_to_float(dy[i]);
        if (y != nullptr && !(pd_to_float(y[i]) > 0.f)) g = 0.f;
        if (dx != nullptr) dx[i] = pd_from_float<T>(g);
        acc += g;
      }
    }
    if (C <= kThreads) {
      if (active) sm[lane * C + col] = acc;
      __syncthreads();
      if (threadIdx.x < C) {
        float s = 0.f;
        for (int l = 0; l < lanes; ++l) s += sm[l * C + threadIdx.x];
        partial[(int64_t)blockIdx.x * C + threadIdx.x] = s;
      }
      __syncthreads();
    } else if (col < C) {
      partial[(int64_t)blockIdx.x * C + col] = acc;
    }
  }
}

__global__ void __launch_bounds__(kThreads)
colsum_final_kernel(const float* __restrict__ partial, int nblocks, int C, float* __restrict__ out,
                    int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[(int64_t)b * C + c];
  out[c] = accumulate ? out[c] + s : s;
}

// ---- 2x2 stride-2 max-pool on padded NHWC -----------------------------------
// out_mode 0: padded NHWC output; 1: contiguous NCHW output.
template <typename T, typename IdxT>
__global__ void __launch_bounds__(kThreads)
maxpool2_fwd_kernel(const T* __restrict__ x, int N, int C, int H, int W, T* __restrict__ y,
                    int out_mode) {
  const int Ho = H / 2, Wo = W / 2;
  const int Hp = H + 2, Wp = W + 2, Hop = Ho + 2, Wop = Wo + 2;
  const IdxT step = (IdxT)gridDim.x * blockDim.x;
  const IdxT row = (IdxT)Wp * C;
  if (out_mode == 0) {
    const IdxT total = (IdxT)N * Hop * Wop * C;
    for (IdxT i = (IdxT)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
      const IdxT p = i / (IdxT)C, q = p / (IdxT)Wop, n = q / (IdxT)Hop;
      const int c = (int)(i - p * C), wo = (int)(p - q * Wop), ho = (int)(q - n * Hop);
      float m = 0.f;
      if (ho >= 1 && ho <= Ho && wo >= 1 && wo <= Wo) {
        const T* b = x + ((n * Hp + (IdxT)(2 * ho - 1)) * Wp + (IdxT)(2 * wo - 1)) * C + c;
        m = fmaxf(fmaxf(pd_to_float(b[0]), pd_to_float(b[C])), fmaxf(pd_to_float(b[row]), pd_to_float(b[row + C])));
      }
      y[i] = pd_from_float<T>(m);
    }
  } else {
    const IdxT total = (IdxT)N * C * Ho * Wo;
    // iterate in NHWC order for coalesced reads; small tensors only use this mode
    for (IdxT i = (IdxT)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
      const IdxT p = i / (IdxT)C, q = p / (IdxT)Wo, n = q / (IdxT)Ho;
      const int c = (int)(i - p * C), wo = (int)(p - q * Wo), ho = (int)(q - n * Ho);
      const T* b = x + ((n * Hp + (IdxT)(2 * ho + 1)) * Wp + (IdxT)(2 * wo + 1)) * C + c;
      float m = fmaxf(fmaxf(pd_to_float(b[0]), pd_to_float(b[C])), fmaxf(pd_to_float(b[row]), pd_to_float(b[row + C])));
      y[((n * C + c) * Ho + (IdxT)ho) * Wo + wo] = pd_from_float<T>(m);
    }
  }
}

// dx (padded NHWC, incl. zero border) from dy.  The gradient goes to the first
// maximum of the window in (h,w) scan order, as ATen's max_pool2d does.
// dy_mode 0: dy is padded NHWC; 1: dy is contiguous NCHW.
// relu_mask != 0: x is a ReLU output and dx is additionally multiplied by (x > 0).
template <typename T, typename IdxT>
__global__ void __launch_bounds__(kThreads)
maxpool2_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, int N, int C, int H, int W,
                    T* __restrict__ dx, int dy_mode, int relu_mask) {
  const int Ho = H / 2, Wo = W / 2;
  const int Hp = H + 2, Wp = W + 2, Hop = Ho + 2, Wop = Wo + 2;
  const IdxT total = (IdxT)N * Hp * Wp * C;
  const IdxT step = (IdxT)gridDim.x * blockDim.x;
  const IdxT row = (IdxT)Wp * C;
  for (IdxT i = (IdxT)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const IdxT p = i / (IdxT)C, q = p / (IdxT)Wp, n = q / (IdxT)Hp;
    const int c = (int)(i - p * C), wp = (int)(p - q * Wp), hp = (int)(q - n * Hp);
    float g = 0.f;
    const int h = hp - 1, w = wp - 1;
    if (h >= 0 && w >= 0 && h < 2 * Ho && w < 2 * Wo) {
      const int ho = h >> 1, wo = w >> 1;
      const T* b = x + ((n * Hp + (IdxT)(2 * ho + 1)) * Wp + (IdxT)(2 * wo + 1)) * C + c;
      const float v00 = pd_to_float(b[0]), v01 = pd_to_float(b[C]);
      const float v10 = pd_to_float(b[row]), v11 = pd_to_float(b[row + C]);
      int arg = 0; float m = v00;
      if (v01 > m) { m = v01; arg = 1; }
      if (v10 > m) { m = v10; arg = 2; }
      if (v11 > m) { m = v11; arg = 3; }
      const int me = ((h & 1) << 1) | (w & 1);
      if (me == arg && !(relu_mask && !(m > 0.f))) {
        g = dy_mode == 0
                ? pd_to_float(dy[((n * Hop + (IdxT)(ho + 1)) * Wop + (IdxT)(wo + 1)) * C + c])
                : pd_to_float(dy[((n * C + c) * Ho + (IdxT)ho) * Wo + wo]);
      }
    }
    dx[i] = pd_from_float<T>(g);
  }
}

// ---- dropout (counter-based RNG; mask kept as bytes) -------------------------
__device__ __forceinline__ uint32_t mix32(uint64_t k) {
  // splitmix64 finaliser; one draw per element index and (seed, offset) pair
  k += 0x9E3779B97F4A7C15ull;
  k = (k ^ (k >> 30)) * 0xBF58476D1CE4E5B9ull;
  k = (k ^ (k >> 27)) * 0x94D049BB133111EBull;
  k = k ^ (k >> 31);
  return (uint32_t)(k >> 32);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
dropout_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint8_t* __restrict__ mask, int64_t n,
                   float p, uint64_t seed, uint64_t offset) {
  const float scale = 1.f / (1.f - p);
  const uint32_t thresh = (uint32_t)((double)p * 4294967296.0 > 4294967295.0 ? 4294967295.0
                                                                            : (double)p * 4294967296.0);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t r = mix32((seed * 0x100000001B3ull) ^ (offset + (uint64_t)i));
    const uint8_t keep = r >= thresh;
    mask[i] = keep;
    y[i] = keep ? pd_from_float<T>(pd_to_float(x[i]) * scale) : pd_from_float<T>(0.f);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
dropout_bwd_kernel(const T* __restrict__ dy, const uint8_t* __restrict__ mask, T* __restrict__ dx,
                   int64_t n, float p) {
  const float scale = 1.f / (1.f - p);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    dx[i] = mask[i] ? pd_from_float<T>(pd_to_float(dy[i]) * scale) : pd_from_float<T>(0.f);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
add_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    y[i] = pd_from_float<T>(pd_to_float(a[i]) + pd_to_float(b[i]));
}


// ---- bf16 x 8 (16-byte) variants of the hot layout kernels --------------------
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x; f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
  return v;
}

__global__ void __launch_bounds__(kThreads)
add_bf16x8_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ y, int64_t nvec) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float fa[8], fb[8];
    const uint4 va = a[i], vb = b[i];
    unpack8(va, fa);
    unpack8(vb, fb);
#pragma unroll
    for (int k = 0; k < 8; ++k) fa[k] += fb[k];
    y[i] = pack8(fa);
  }
}
__device__ __forceinline__ uint4 max8(const uint4& a, const uint4& b) {
  uint4 r;
  const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* y = reinterpret_cast<const __nv_bfloat162*>(&b);
  __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j] = __hmax2(x[j], y[j]);
  return r;
}

// padded NHWC -> padded NHWC, 8 channels per thread.  IdxT: uint32_t when every vector index of x and y fits
// (64-bit divisions cost more than the memory accesses of these kernels), int64_t otherwise.
template <typename IdxT>
__global__ void __launch_bounds__(kThreads)
maxpool2_fwd_bf16x8_kernel(const uint4* __restrict__ x, int N, int C8, int H, int W, uint4* __restrict__ y) {
  const int Ho = H / 2, Wo = W / 2;
  const int Hp = H + 2, Wp = W + 2, Hop = Ho + 2, Wop = Wo + 2;
  const IdxT total = (IdxT)N * Hop * Wop * C8;
  const IdxT step = (IdxT)gridDim.x * blockDim.x;
  const IdxT row = (IdxT)Wp * C8;
  for (IdxT i = (IdxT)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const IdxT p = i / (IdxT)C8, q = p / (IdxT)Wop, n = q / (IdxT)Hop;
    const int c = (int)(i - p * C8), wo = (int)(p - q * Wop), ho = (int)(q - n * Hop);
    uint4 m = make_uint4(0, 0, 0, 0);
    if (ho >= 1 && ho <= Ho && wo >= 1 && wo <= Wo) {
      const uint4* b = x + ((n * Hp + (IdxT)(2 * ho - 1)) * Wp + (IdxT)(2 * wo - 1)) * C8 + c;
      m = max8(max8(b[0], b[C8]), max8(b[row], b[row + C8]));
    }
    y[i] = m;
  }
}

// One thread per (output window, 8 channels): reads the 2x2 window and dy once, writes the four
// dx vectors.  The padded border of dx is written by the threads of the border windows.
__global__ void __launch_bounds__(kThreads)
maxpool2_bwd_bf16x8_kernel(const uint4* __restrict__ x, const uint4* __restrict__ dy, int N, int C8, int H, int W,
                           uint4* __restrict__ dx, int relu_mask) {
  const int Ho = H / 2, Wo = W / 2;
  const int Hp = H + 2, Wp = W + 2, Hop = Ho + 2, Wop = Wo + 2;
  // windows cover padded rows/cols pairwise: window (i, j), i in [0, Ho], j in [0, Wo], owns padded pixels
  // (2i, 2j) .. (2i+1, 2j+1); interior pooling windows are the pixels (2ho+1.., 2wo+1..), i.e. shifted by one,
  // so here a thread is assigned to a pooling window (ho, wo) in [-1.., ..]: simpler to loop over pooling
  // windows for the interior and let a second pass zero the border.
  const int64_t total = (int64_t)N * Ho * Wo * C8;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C8);
    const int64_t p = i / C8;
    const int wo = (int)(p % Wo), ho = (int)((p / Wo) % Ho), n = (int)(p / ((int64_t)Wo * Ho));
    const int64_t base = (((int64_t)n * Hp + (2 * ho + 1)) * Wp + (2 * wo + 1)) * C8 + c;
    float v[4][8], g[8];
    unpack8(x[base], v[0]);
    unpack8(x[base + C8], v[1]);
    unpack8(x[base + (int64_t)Wp * C8], v[2]);
    unpack8(x[base + (int64_t)Wp * C8 + C8], v[3]);
    unpack8(dy[(((int64_t)n * Hop + ho + 1) * Wop + wo + 1) * C8 + c], g);
    float o[4][8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      int arg = 0; float m = v[0][k];
      if (v[1][k] > m) { m = v[1][k]; arg = 1; }
      if (v[2][k] > m) { m = v[2][k]; arg = 2; }
      if (v[3][k] > m) { m = v[3][k]; arg = 3; }
      const float gg = (relu_mask && !(m > 0.f)) ? 0.f : g[k];
#pragma unroll
      for (int q = 0; q < 4; ++q) o[q][k] = (q == arg) ? gg : 0.f;
    }
    dx[base] = pack8(o[0]);
    dx[base + C8] = pack8(o[1]);
    dx[base + (int64_t)Wp * C8] = pack8(o[2]);
    dx[base + (int64_t)Wp * C8 + C8] = pack8(o[3]);
  }
  // border pixels (and odd trailing rows/cols, which no window covers) are zero
  const int64_t border = (int64_t)N * Hp * Wp * C8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < border;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t p = i / C8;
    const int wp = (int)(p % Wp), hp = (int)((p / Wp) % Hp);
    if (hp == 0 || wp == 0 || hp > 2 * Ho || wp > 2 * Wo) dx[i] = zero;
  }
}

// dx = dy * (y > 0), 8 columns per thread, plus per-block column partial sums (C % 8 == 0, C8 <= kThreads).
__global__ void __launch_bounds__(kThreads)
relu_bwd_colsum_bf16x8_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ y, uint4* __restrict__ dx,
                              int64_t rows, int C8, float* __restrict__ partial) {
  extern __shared__ float sm[];   // [lanes][C8 * 8]
  const int lanes = kThreads / C8;
  const int lane = threadIdx.x / C8, c = threadIdx.x % C8;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  if (lane < lanes) {
    for (int64_t r = (int64_t)blockIdx.x * lanes + lane; r < rows; r += (int64_t)gridDim.x * lanes) {
      const int64_t i = r * C8 + c;
      float g[8];
      unpack8(dy[i], g);
      if (y != nullptr) {
        float yv[8];
        unpack8(y[i], yv);
#pragma unroll
        for (int k = 0; k < 8; ++k) if (!(yv[k] > 0.f)) g[k] = 0.f;
      }
      if (dx != nullptr) dx[i] = pack8(g);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += g[k];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) sm[(lane * C8 + c) * 8 + k] = acc[k];
  }
  __syncthreads();
  const int C = C8 * 8;
  for (int col = threadIdx.x; col < C; col += blockDim.x) {
    float s = 0.f;
    for (int l = 0; l < lanes; ++l) s += sm[l * C + col];
    partial[(int64_t)blockIdx.x * C + col] = s;
  }
}

// The same for wide matrices (C8 > kThreads): blockIdx.y picks a chunk of kThreads 16-byte columns, blockIdx.x strides
// over the rows; a thread keeps the sums of its 8 columns in registers and writes them straight to partial[x][C].
__global__ void __launch_bounds__(kThreads)
relu_bwd_colsum_wide_bf16x8_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ y, uint4* __restrict__ dx,
                                   int64_t rows, int C8, float* __restrict__ partial) {
  const int cv = blockIdx.y * kThreads + threadIdx.x;
  if (cv >= C8) return;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const int64_t i = r * C8 + cv;
    float g[8];
    unpack8(dy[i], g);
    if (y != nullptr) {
      float yv[8];
      unpack8(y[i], yv);
#pragma unroll
      for (int k = 0; k < 8; ++k) if (!(yv[k] > 0.f)) g[k] = 0.f;
    }
    if (dx != nullptr) dx[i] = pack8(g);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] += g[k];
  }
  float4* o = reinterpret_cast<float4*>(partial + (int64_t)blockIdx.x * C8 * 8 + (int64_t)cv * 8);
  o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// out[c] (+)= sum_b partial[b][c].  The partial rows are a few hundred to a thousand and C is small, so the kernel is
// a latency chain unless the rows are spread wide: 8 columns per block, 128 threads per column (four warps, each
// lane summing every 128th row with independent loads), a shuffle tree per warp and one thread per column at the end.
__global__ void __launch_bounds__(1024)
colsum_final_fast_kernel(const float* __restrict__ partial, int nblocks, int C, float* __restrict__ out,
                         int accumulate) {
  __shared__ float sm[8][4];
  const int col = threadIdx.x >> 7, r = threadIdx.x & 127;
  const int c = blockIdx.x * 8 + col;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (c < C) {
    int b = r;
    for (; b + 384 < nblocks; b += 512) {
      s0 += partial[(int64_t)b * C + c];
      s1 += partial[(int64_t)(b + 128) * C + c];
      s2 += partial[(int64_t)(b + 256) * C + c];
      s3 += partial[(int64_t)(b + 384) * C + c];
    }
    for (; b < nblocks; b += 128) s0 += partial[(int64_t)b * C + c];
  }
  float s = (s0 + s1) + (s2 + s3);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) sm[col][r >> 5] = s;
  __syncthreads();
  if (r == 0 && c < C) {
    const float t = (sm[col][0] + sm[col][1]) + (sm[col][2] + sm[col][3]);
    out[c] = accumulate ? out[c] + t : t;
  }
}

// im2col for small C: one thread per padded pixel row, Kpad bf16 written as 16-byte vectors.
template <typename S>
__global__ void __launch_bounds__(kThreads)
im2col3x3_rows_kernel(const S* __restrict__ src, int64_t sN, int64_t sC, int64_t sH, int64_t sW,
                      int N, int C, int H, int W, int Kpad, __nv_bfloat16* __restrict__ dst) {
  const int Hp = H + 2, Wp = W + 2;
  const int64_t rows = (int64_t)N * Hp * Wp;
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < rows;
       p += (int64_t)gridDim.x * blockDim.x) {
    const int wp = (int)(p % Wp);
    const int hp = (int)((p / Wp) % Hp);
    const int n = (int)(p / ((int64_t)Wp * Hp));
    const bool inside = hp >= 1 && hp <= H && wp >= 1 && wp <= W;
    uint4* out = reinterpret_cast<uint4*>(dst + p * Kpad);
    for (int k0 = 0; k0 < Kpad; k0 += 8) {
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = k0 + j;
        float v = 0.f;
        if (inside && k < 9 * C) {
          const int t = k / C, c = k - t * C;
          const int h = hp - 1 + t / 3 - 1, w = wp - 1 + t % 3 - 1;
          if (h >= 0 && h < H && w >= 0 && w < W) v = pd_to_float(src[n * sN + c * sC + h * sH + w * sW]);
        }
        f[j] = v;
      }
      out[k0 >> 3] = pack8(f);
    }
  }
}

// The same for C == 3 (the first layer of the image models).  One block per padded pixel row (n, hp): the three
// source rows of the three channels are staged in shared memory with a zero halo (nine coalesced row reads serve
// the 27 values of every pixel of the row), then each thread assembles 8 patch columns of a pixel and writes them
// as one 16-byte vector, a warp writing 512 contiguous bytes.
template <typename S>
__global__ void __launch_bounds__(kThreads)
im2col3x3_c3_kernel(const S* __restrict__ src, int64_t sN, int64_t sC, int64_t sH, int64_t sW,
                    int N, int H, int W, int K8, uint4* __restrict__ dst) {
  extern __shared__ float rows_sm[];          // [3 channels][3 rows][W + 2]
  const int Hp = H + 2, Wp = W + 2;
  const int rows = N * Hp;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const int n = row / Hp, hp = row - n * Hp;
    uint4* out = dst + (int64_t)row * Wp * K8;
    if (hp == 0 || hp == Hp - 1) {
      for (int i = threadIdx.x; i < Wp * K8; i += blockDim.x) out[i] = zero;
      continue;
    }
    __syncthreads();                          // the previous row's readers are done
    for (int i0 = 0; i0 < 9 * Wp; i0 += 8 * kThreads) {
      float v[8];                                          // eight loads in flight per thread
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * kThreads + threadIdx.x;
        const int cr = i / Wp, col = i - cr * Wp;          // cr = c * 3 + r
        const int c = cr / 3, r = cr - c * 3;
        const int h = hp - 2 + r, w = col - 1;
        v[u] = 0.f;
        if (i < 9 * Wp && h >= 0 && h < H && w >= 0 && w < W)
          v[u] = pd_to_float(src[(int64_t)n * sN + c * sC + h * sH + w * sW]);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * kThreads + threadIdx.x;
        if (i < 9 * Wp) rows_sm[i] = v[u];
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < Wp * K8; i += blockDim.x) {
      const int wp = i / K8, q = i - wp * K8;
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
      if (wp >= 1 && wp <= W && q * 8 < 27) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int k = q * 8 + j;
          const int t = k / 3, c = k - t * 3;
          const int r = t / 3, sx = t - r * 3;
          if (k < 27) f[j] = rows_sm[(c * 3 + r) * Wp + wp - 1 + sx];
        }
      }
      out[i] = pack8(f);
    }
  }
}

// Max-pool backward with the bias-gradient reduction of the producing convolution folded in: besides dx, every
// block leaves the column sums of the gradient it routed in partial[blockIdx.x][C] (the column sums of dx are the
// sums of the routed values).  H and W even; gridDim.x * kThreads is a multiple of C8, so a thread stays on one
// group of 8 channels; the border of dx is enumerated directly (2 * Wp + 2 * H pixels per image).
template <typename IdxT>
__global__ void __launch_bounds__(kThreads)
maxpool2_bwd_colsum_bf16x8_kernel(const uint4* __restrict__ x, const uint4* __restrict__ dy, int N, int C8, int H,
                                  int W, uint4* __restrict__ dx, int relu_mask, float* __restrict__ partial) {
  extern __shared__ float sm[];   // [kThreads / C8][C8 * 8] when partial != nullptr
  const int Ho = H / 2, Wo = W / 2;
  const int Hp = H + 2, Wp = W + 2, Hop = Ho + 2, Wop = Wo + 2;
  const IdxT total = (IdxT)N * Ho * Wo * C8;
  const IdxT step = (IdxT)gridDim.x * blockDim.x;
  const IdxT row = (IdxT)Wp * C8;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  for (IdxT i = (IdxT)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const IdxT p = i / (IdxT)C8, q2 = p / (IdxT)Wo, n = q2 / (IdxT)Ho;
    const int c = (int)(i - p * C8), wo = (int)(p - q2 * Wo), ho = (int)(q2 - n * Ho);
    const IdxT base = ((n * Hp + (IdxT)(2 * ho + 1)) * Wp + (IdxT)(2 * wo + 1)) * C8 + c;
    float v[4][8], g[8];
    unpack8(x[base], v[0]);
    unpack8(x[base + C8], v[1]);
    unpack8(x[base + row], v[2]);
    unpack8(x[base + row + C8], v[3]);
    unpack8(dy[((n * Hop + (IdxT)(ho + 1)) * Wop + (IdxT)(wo + 1)) * C8 + c], g);
    float o[4][8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      int arg = 0; float m = v[0][k];
      if (v[1][k] > m) { m = v[1][k]; arg = 1; }
      if (v[2][k] > m) { m = v[2][k]; arg = 2; }
      if (v[3][k] > m) { m = v[3][k]; arg = 3; }
      const float gg = (relu_mask && !(m > 0.f)) ? 0.f : g[k];
      acc[k] += gg;
#pragma unroll
      for (int q = 0; q < 4; ++q) o[q][k] = (q == arg) ? gg : 0.f;
    }
    dx[base] = pack8(o[0]);
    dx[base + C8] = pack8(o[1]);
    dx[base + row] = pack8(o[2]);
    dx[base + row + C8] = pack8(o[3]);
  }
  const int per_image = 2 * Wp + 2 * H;
  const IdxT border = (IdxT)N * per_image * C8;
  for (IdxT i = (IdxT)blockIdx.x * blockDim.x + threadIdx.x; i < border; i += step) {
    const IdxT p = i / (IdxT)C8, n = p / (IdxT)per_image;
    const int c = (int)(i - p * C8), b = (int)(p - n * per_image);
    int hp, wp;
    if (b < Wp) { hp = 0; wp = b; }
    else if (b < 2 * Wp) { hp = Hp - 1; wp = b - Wp; }
    else { const int r = b - 2 * Wp; hp = 1 + (r >> 1); wp = (r & 1) ? Wp - 1 : 0; }
    dx[((n * Hp + (IdxT)hp) * Wp + (IdxT)wp) * C8 + c] = zero;
  }
  if (partial != nullptr) {
    // a thread's channel group: (blockIdx.x * kThreads + threadIdx.x) % C8 == threadIdx.x % C8 (kThreads % C8 == 0)
    const int lanes = kThreads / C8, lane = threadIdx.x / C8, c = threadIdx.x % C8;
#pragma unroll
    for (int k = 0; k < 8; ++k) sm[(lane * C8 + c) * 8 + k] = acc[k];
    __syncthreads();
    const int C = C8 * 8;
    for (int col = threadIdx.x; col < C; col += blockDim.x) {
      float s = 0.f;
      for (int l = 0; l < lanes; ++l) s += sm[l * C + col];
      partial[(int64_t)blockIdx.x * C + col] = s;
    }
  }
}

}  // namespace

#define PD_DISPATCH_T(dtype, ...)                                   \
  if (dtype == PD_F32) { using T = float; __VA_ARGS__ }             \
  else if (dtype == PD_BF16) { using T = __nv_bfloat16; __VA_ARGS__ } \
  else { pd_set_error("bad dtype %d", dtype); return PD_ERR_INVALID; }

PD_EXPORT int pd_pack_pnhwc(const void* src, int src_dtype, int64_t sN, int64_t sC, int64_t sH,
                            int64_t sW, int N, int C, int H, int W, void* dst, int dst_dtype,
                            void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(src && dst && N > 0 && C > 0 && H > 0 && W > 0, "pd_pack_pnhwc: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  int grid = grid_cap((int64_t)N * (H + 2), 16);
  if (src_dtype == PD_F32 && dst_dtype == PD_F32)
    pack_pnhwc_kernel<float, float><<<grid, kThreads, 0, s>>>((const float*)src, sN, sC, sH, sW, N, C, H, W, (float*)dst);
  else if (src_dtype == PD_F32 && dst_dtype == PD_BF16)
    pack_pnhwc_kernel<float, __nv_bfloat16><<<grid, kThreads, 0, s>>>((const float*)src, sN, sC, sH, sW, N, C, H, W, (__nv_bfloat16*)dst);
  else if (src_dtype == PD_BF16 && dst_dtype == PD_BF16)
    pack_pnhwc_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)src, sN, sC, sH, sW, N, C, H, W, (__nv_bfloat16*)dst);
  else if (src_dtype == PD_BF16 && dst_dtype == PD_F32)
    pack_pnhwc_kernel<__nv_bfloat16, float><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)src, sN, sC, sH, sW, N, C, H, W, (float*)dst);
  else PD_REQUIRE(false, "pd_pack_pnhwc: bad dtype");
  PD_LAUNCH_CHECK("pack_pnhwc_kernel");
  return PD_OK;
}

PD_EXPORT int pd_unpack_pnhwc(const void* src, int src_dtype, int N, int C, int H, int W, void* dst,
                              int dst_dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(src && dst && N > 0 && C > 0 && H > 0 && W > 0, "pd_unpack_pnhwc: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  int grid = grid_cap((int64_t)N * H, 16);
  if (src_dtype == PD_F32 && dst_dtype == PD_F32)
    unpack_pnhwc_kernel<float, float><<<grid, kThreads, 0, s>>>((const float*)src, N, C, H, W, (float*)dst);
  else if (src_dtype == PD_BF16 && dst_dtype == PD_BF16)
    unpack_pnhwc_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)src, N, C, H, W, (__nv_bfloat16*)dst);
  else if (src_dtype == PD_BF16 && dst_dtype == PD_F32)
    unpack_pnhwc_kernel<__nv_bfloat16, float><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)src, N, C, H, W, (float*)dst);
  else if (src_dtype == PD_F32 && dst_dtype == PD_BF16)
    unpack_pnhwc_kernel<float, __nv_bfloat16><<<grid, kThreads, 0, s>>>((const float*)src, N, C, H, W, (__nv_bfloat16*)dst);
  else PD_REQUIRE(false, "pd_unpack_pnhwc: bad dtype");
  PD_LAUNCH_CHECK("unpack_pnhwc_kernel");
  return PD_OK;
}

PD_EXPORT int pd_im2col3x3(const void* src, int src_dtype, int64_t sN, int64_t sC, int64_t sH,
                           int64_t sW, int N, int C, int H, int W, int Kpad, void* dst,
                           int dst_dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(src && dst && N > 0 && C > 0 && H > 0 && W > 0 && Kpad >= 9 * C, "pd_im2col3x3: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  int64_t total = (int64_t)N * (H + 2) * (W + 2) * Kpad;
  int grid = grid_cap((total + kThreads - 1) / kThreads, 16);
  if (dst_dtype == PD_BF16 && (Kpad % 8) == 0 && ((uintptr_t)dst % 16) == 0) {
    const int64_t rows = (int64_t)N * (H + 2) * (W + 2);
    const size_t sm3 = (size_t)9 * (W + 2) * sizeof(float);
    if (C == 3 && sm3 <= 48 * 1024 && rows * (Kpad / 8) < (1ll << 31)) {
      const int K8 = Kpad / 8;
      const int g3 = (int)std::min<int64_t>((int64_t)N * (H + 2), 1 << 20);   // one padded row per block
      if (src_dtype == PD_F32)
        im2col3x3_c3_kernel<float><<<g3, kThreads, sm3, s>>>((const float*)src, sN, sC, sH, sW, N, H, W, K8, (uint4*)dst);
      else
        im2col3x3_c3_kernel<__nv_bfloat16><<<g3, kThreads, sm3, s>>>((const __nv_bfloat16*)src, sN, sC, sH, sW, N, H, W, K8, (uint4*)dst);
      PD_LAUNCH_CHECK("im2col3x3_c3_kernel");
      return PD_OK;
    }
    const int g2 = grid_cap((rows + kThreads - 1) / kThreads, 16);
    if (src_dtype == PD_F32)
      im2col3x3_rows_kernel<float><<<g2, kThreads, 0, s>>>((const float*)src, sN, sC, sH, sW, N, C, H, W, Kpad, (__nv_bfloat16*)dst);
    else
      im2col3x3_rows_kernel<__nv_bfloat16><<<g2, kThreads, 0, s>>>((const __nv_bfloat16*)src, sN, sC, sH, sW, N, C, H, W, Kpad, (__nv_bfloat16*)dst);
    PD_LAUNCH_CHECK("im2col3x3_rows_kernel");
    return PD_OK;
  }
  if (src_dtype == PD_F32 && dst_dtype == PD_F32)
    im2col3x3_kernel<float, float><<<grid, kThreads, 0, s>>>((const float*)src, sN, sC, sH, sW, N, C, H, W, Kpad, (float*)dst);
  else if (src_dtype == PD_F32 && dst_dtype == PD_BF16)
    im2col3x3_kernel<float, __nv_bfloat16><<<grid, kThreads, 0, s>>>((const float*)src, sN, sC, sH, sW, N, C, H, W, Kpad, (__nv_bfloat16*)dst);
  else if (src_dtype == PD_BF16 && dst_dtype == PD_BF16)
    im2col3x3_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)src, sN, sC, sH, sW, N, C, H, W, Kpad, (__nv_bfloat16*)dst);
  else PD_REQUIRE(false, "pd_im2col3x3: bad dtype combination");
  PD_LAUNCH_CHECK("im2col3x3_kernel");
  return PD_OK;
}

PD_EXPORT int pd_relu_fwd(const void* x, void* y, int64_t n, int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x && y && n >= 0, "pd_relu_fwd: bad arguments");
  if (n == 0) return PD_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PD_BF16 && (n % 8) == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0) {
    int64_t n8 = n / 8;
    relu_fwd_bf16x8_kernel<<<grid_cap((n8 + kThreads - 1) / kThreads), kThreads, 0, s>>>((const uint4*)x, (uint4*)y, n8);
  } else {
    PD_DISPATCH_T(dtype, relu_fwd_kernel<T><<<grid_cap((n + kThreads - 1) / kThreads), kThreads, 0, s>>>((const T*)x, (T*)y, n);)
  }
  PD_LAUNCH_CHECK("relu_fwd_kernel");
  return PD_OK;
}

PD_EXPORT int pd_relu_bwd(const void* dy, const void* y, void* dx, int64_t n, int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(dy && y && dx && n >= 0, "pd_relu_bwd: bad arguments");
  if (n == 0) return PD_OK;
  cudaStream_t s = (cudaStream_t)stream;
  PD_DISPATCH_T(dtype, relu_bwd_kernel<T><<<grid_cap((n + kThreads - 1) / kThreads), kThreads, 0, s>>>((const T*)dy, (const T*)y, (T*)dx, n);)
  PD_LAUNCH_CHECK("relu_bwd_kernel");
  return PD_OK;
}

// workspace: at least pd_colsum_workspace_bytes(C) bytes of device memory.
PD_EXPORT int64_t pd_colsum_workspace_bytes(int C) {
  return (int64_t)pd_num_sms() * 8 * (int64_t)C * sizeof(float);   // >= blocks launched x C floats
}

PD_EXPORT int pd_relu_bwd_colsum(const void* dy, const void* y, void* dx, int64_t rows, int C,
                                 int dtype, float* colsum, int accumulate, void* workspace,
                                 int64_t workspace_bytes, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(dy && colsum && workspace && rows >= 0 && C > 0, "pd_relu_bwd_colsum: bad arguments");
  PD_REQUIRE(C <= kThreads ? (kThreads / C) * C * (int)sizeof(float) <= 48 * 1024 : true, "pd_relu_bwd_colsum: C too large");
  PD_REQUIRE(workspace_bytes >= pd_colsum_workspace_bytes(C), "pd_relu_bwd_colsum: workspace too small");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PD_BF16 && (C % 8) == 0 && C / 8 <= kThreads && ((uintptr_t)dy % 16) == 0 &&
      (y == nullptr || ((uintptr_t)y % 16) == 0) && (dx == nullptr || ((uintptr_t)dx % 16) == 0)) {
    const int C8 = C / 8, lanes8 = kThreads / C8;
    int g8 = grid_cap((rows + lanes8 - 1) / lanes8, 8);
    relu_bwd_colsum_bf16x8_kernel<<<g8, kThreads, (size_t)lanes8 * C * sizeof(float), s>>>(
        (const uint4*)dy, (const uint4*)y, (uint4*)dx, rows, C8, (float*)workspace);
    PD_LAUNCH_CHECK("relu_bwd_colsum_bf16x8_kernel");
    colsum_final_fast_kernel<<<(C + 7) / 8, 1024, 0, s>>>((const float*)workspace, g8, C, colsum, accumulate);
    PD_LAUNCH_CHECK("colsum_final_fast_kernel");
    return PD_OK;
  }
  if (dtype == PD_BF16 && (C % 8) == 0 && C / 8 > kThreads && ((uintptr_t)dy % 16) == 0 &&
      (y == nullptr || ((uintptr_t)y % 16) == 0) && (dx == nullptr || ((uintptr_t)dx % 16) == 0)) {
    const int C8 = C / 8, chunks = (C8 + kThreads - 1) / kThreads;
    int gx = grid_cap(rows, 4) / chunks;
    if (gx < 1) gx = 1;
    relu_bwd_colsum_wide_bf16x8_kernel<<<dim3((unsigned)gx, (unsigned)chunks), kThreads, 0, s>>>(
        (const uint4*)dy, (const uint4*)y, (uint4*)dx, rows, C8, (float*)workspace);
    PD_LAUNCH_CHECK("relu_bwd_colsum_wide_bf16x8_kernel");
    colsum_final_fast_kernel<<<(C + 7) / 8, 1024, 0, s>>>((const float*)workspace, gx, C, colsum, accumulate);
    PD_LAUNCH_CHECK("colsum_final_fast_kernel");
    return PD_OK;
  }
  int lanes = C <= kThreads ? kThreads / C : 1;
  int64_t want = (rows + lanes - 1) / lanes;
  int grid = grid_cap(want, 4);
  size_t smem = C <= kThreads ? (size_t)lanes * C * sizeof(float) : 0;
  PD_DISPATCH_T(dtype, relu_bwd_colsum_kernel<T><<<grid, kThreads, smem, s>>>((const T*)dy, (const T*)y, (T*)dx, rows, C, (float*)workspace);)
  PD_LAUNCH_CHECK("relu_bwd_colsum_kernel");
  colsum_final_fast_kernel<<<(C + 7) / 8, 1024, 0, s>>>((const float*)workspace, grid, C, colsum, accumulate);
  PD_LAUNCH_CHECK("colsum_final_fast_kernel");
  return PD_OK;
}

PD_EXPORT int pd_maxpool2_fwd(const void* x, int N, int C, int H, int W, void* y, int out_mode,
                              int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x && y && N > 0 && C > 0 && H >= 2 && W >= 2, "pd_maxpool2_fwd: bad arguments");
  PD_REQUIRE(out_mode == 0 || out_mode == 1, "pd_maxpool2_fwd: bad out_mode");
  cudaStream_t s = (cudaStream_t)stream;
  int64_t total = out_mode == 0 ? (int64_t)N * (H / 2 + 2) * (W / 2 + 2) * C : (int64_t)N * C * (H / 2) * (W / 2);
  int grid = grid_cap((total + kThreads - 1) / kThreads, 16);
  if (dtype == PD_BF16 && out_mode == 0 && (C % 8) == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0) {
    const int g8 = grid_cap((total / 8 + kThreads - 1) / kThreads, 16);
    if ((int64_t)N * (H + 2) * (W + 2) * (C / 8) < (1ll << 31) - (int64_t)g8 * kThreads)
      maxpool2_fwd_bf16x8_kernel<uint32_t><<<g8, kThreads, 0, s>>>((const uint4*)x, N, C / 8, H, W, (uint4*)y);
    else
      maxpool2_fwd_bf16x8_kernel<int64_t><<<g8, kThreads, 0, s>>>((const uint4*)x, N, C / 8, H, W, (uint4*)y);
    PD_LAUNCH_CHECK("maxpool2_fwd_bf16x8_kernel");
    return PD_OK;
  }
  if ((int64_t)N * (H + 2) * (W + 2) * C < (1ll << 31) - (int64_t)grid * kThreads) {
    PD_DISPATCH_T(dtype, maxpool2_fwd_kernel<T, uint32_t><<<grid, kThreads, 0, s>>>((const T*)x, N, C, H, W, (T*)y, out_mode);)
  } else {
    PD_DISPATCH_T(dtype, maxpool2_fwd_kernel<T, int64_t><<<grid, kThreads, 0, s>>>((const T*)x, N, C, H, W, (T*)y, out_mode);)
  }
  PD_LAUNCH_CHECK("maxpool2_fwd_kernel");
  return PD_OK;
}

namespace {
// 32-bit vector indices are enough (with room for one grid stride past the end)
bool pool_idx32(int N, int C8, int H, int W, int grid) {
  return (int64_t)N * (H + 2) * (W + 2) * C8 < (1ll << 31) - (int64_t)grid * kThreads;
}
bool pool_bwd_fast_ok(const void* x, const void* dy, const void* dx, int C, int H, int W, int dtype) {
  return dtype == PD_BF16 && (C % 8) == 0 && (kThreads % (C / 8)) == 0 && (H % 2) == 0 && (W % 2) == 0 &&
         (((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dx) % 16) == 0;
}
}  // namespace

// Max-pool backward (dy in padded NHWC) that also leaves per-block column sums of dx in `partial`
// (`*partial_rows` rows of C floats, at most pd_colsum_workspace_bytes(C) bytes); pd_colsum_finish adds them up.
PD_EXPORT int pd_maxpool2_bwd_colsum(const void* x, const void* dy, int N, int C, int H, int W, void* dx,
                                     int relu_mask, int dtype, float* partial, int64_t partial_bytes,
                                     int* partial_rows, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x && dy && dx && partial && partial_rows && N > 0 && C > 0 && H >= 2 && W >= 2,
             "pd_maxpool2_bwd_colsum: bad arguments");
  PD_REQUIRE(partial_bytes >= pd_colsum_workspace_bytes(C), "pd_maxpool2_bwd_colsum: partial buffer too small");
  PD_REQUIRE(pool_bwd_fast_ok(x, dy, dx, C, H, W, dtype),
             "pd_maxpool2_bwd_colsum: needs bf16, even H and W, C a multiple of 8 with 256 % (C / 8) == 0, 16-byte pointers");
  cudaStream_t s = (cudaStream_t)stream;
  const int C8 = C / 8;
  const int64_t win = (int64_t)N * (H / 2) * (W / 2) * C8;
  const int grid = grid_cap((win + kThreads - 1) / kThreads, 8);
  if (pool_idx32(N, C8, H, W, grid))
    maxpool2_bwd_colsum_bf16x8_kernel<uint32_t><<<grid, kThreads, (size_t)kThreads * 8 * sizeof(float), s>>>(
        (const uint4*)x, (const uint4*)dy, N, C8, H, W, (uint4*)dx, relu_mask, partial);
  else
    maxpool2_bwd_colsum_bf16x8_kernel<int64_t><<<grid, kThreads, (size_t)kThreads * 8 * sizeof(float), s>>>(
        (const uint4*)x, (const uint4*)dy, N, C8, H, W, (uint4*)dx, relu_mask, partial);
  PD_LAUNCH_CHECK("maxpool2_bwd_colsum_bf16x8_kernel");
  *partial_rows = grid;
  return PD_OK;
}

// out[C] (+)= sum over the rows of partial[rows][C].
PD_EXPORT int pd_colsum_finish(const float* partial, int rows, int C, float* out, int accumulate, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(partial && out && rows > 0 && C > 0, "pd_colsum_finish: bad arguments");
  colsum_final_fast_kernel<<<(C + 7) / 8, 1024, 0, (cudaStream_t)stream>>>(partial, rows, C, out, accumulate);
  PD_LAUNCH_CHECK("colsum_final_fast_kernel");
  return PD_OK;
}

PD_EXPORT int pd_maxpool2_bwd(const void* x, const void* dy, int N, int C, int H, int W, void* dx,
                              int dy_mode, int relu_mask, int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x && dy && dx && N > 0 && C > 0 && H >= 2 && W >= 2, "pd_maxpool2_bwd: bad arguments");
  PD_REQUIRE(dy_mode == 0 || dy_mode == 1, "pd_maxpool2_bwd: bad dy_mode");
  cudaStream_t s = (cudaStream_t)stream;
  int64_t total = (int64_t)N * (H + 2) * (W + 2) * C;
  int grid = grid_cap((total + kThreads - 1) / kThreads, 16);
  if (dy_mode == 0 && pool_bwd_fast_ok(x, dy, dx, C, H, W, dtype)) {
    const int64_t win = (int64_t)N * (H / 2) * (W / 2) * (C / 8);
    const int g8 = grid_cap((win + kThreads - 1) / kThreads, 16);
    if (pool_idx32(N, C / 8, H, W, g8))
      maxpool2_bwd_colsum_bf16x8_kernel<uint32_t><<<g8, kThreads, 0, s>>>(
          (const uint4*)x, (const uint4*)dy, N, C / 8, H, W, (uint4*)dx, relu_mask, nullptr);
    else
      maxpool2_bwd_colsum_bf16x8_kernel<int64_t><<<g8, kThreads, 0, s>>>(
          (const uint4*)x, (const uint4*)dy, N, C / 8, H, W, (uint4*)dx, relu_mask, nullptr);
    PD_LAUNCH_CHECK("maxpool2_bwd_colsum_bf16x8_kernel");
    return PD_OK;
  }
  if (dtype == PD_BF16 && dy_mode == 0 && (C % 8) == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)dy % 16) == 0 &&
      ((uintptr_t)dx % 16) == 0) {
    const int64_t win = (int64_t)N * (H / 2) * (W / 2) * (C / 8);
    maxpool2_bwd_bf16x8_kernel<<<grid_cap((win + kThreads - 1) / kThreads, 16), kThreads, 0, s>>>(
        (const uint4*)x, (const uint4*)dy, N, C / 8, H, W, (uint4*)dx, relu_mask);
    PD_LAUNCH_CHECK("maxpool2_bwd_bf16x8_kernel");
    return PD_OK;
  }
  if (total < (1ll << 31) - (int64_t)grid * kThreads) {
    PD_DISPATCH_T(dtype, maxpool2_bwd_kernel<T, uint32_t><<<grid, kThreads, 0, s>>>((const T*)x, (const T*)dy, N, C, H, W, (T*)dx, dy_mode, relu_mask);)
  } else {
    PD_DISPATCH_T(dtype, maxpool2_bwd_kernel<T, int64_t><<<grid, kThreads, 0, s>>>((const T*)x, (const T*)dy, N, C, H, W, (T*)dx, dy_mode, relu_mask);)
  }
  PD_LAUNCH_CHECK("maxpool2_bwd_kernel");
  return PD_OK;
}

PD_EXPORT int pd_dropout_fwd(const void* x, void* y, uint8_t* mask, int64_t n, float p,
                             uint64_t seed, uint64_t offset, int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(x && y && mask && n >= 0 && p >= 0.f && p < 1.f, "pd_dropout_fwd: bad arguments");
  if (n == 0) return PD_OK;
  cudaStream_t s = (cudaStream_t)stream;
  PD_DISPATCH_T(dtype, dropout_fwd_kernel<T><<<grid_cap((n + kThreads - 1) / kThreads), kThreads, 0, s>>>((const T*)x, (T*)y, mask, n, p, seed, offset);)
  PD_LAUNCH_CHECK("dropout_fwd_kernel");
  return PD_OK;
}

PD_EXPORT int pd_dropout_bwd(const void* dy, const uint8_t* mask, void* dx, int64_t n, float p,
                             int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(dy && dx && mask && n >= 0 && p >= 0.f && p < 1.f, "pd_dropout_bwd: bad arguments");
  if (n == 0) return PD_OK;
  cudaStream_t s = (cudaStream_t)stream;
  PD_DISPATCH_T(dtype, dropout_bwd_kernel<T><<<grid_cap((n + kThreads - 1) / kThreads), kThreads, 0, s>>>((const T*)dy, mask, (T*)dx, n, p);)
  PD_LAUNCH_CHECK("dropout_bwd_kernel");
  return PD_OK;
}

PD_EXPORT int pd_add(const void* a, const void* b, void* y, int64_t n, int dtype, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(a && b && y && n >= 0, "pd_add: bad arguments");
  if (n == 0) return PD_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const bool aligned = (((uintptr_t)a | (uintptr_t)b | (uintptr_t)y) & 15) == 0;
  if (dtype == PD_BF16 && aligned && (n % 8) == 0) {
    add_bf16x8_kernel<<<grid_cap((n / 8 + kThreads - 1) / kThreads), kThreads, 0, s>>>((const uint4*)a, (const uint4*)b, (uint4*)y, n / 8);
  } else {
    PD_DISPATCH_T(dtype, add_kernel<T><<<grid_cap((n + kThreads - 1) / kThreads), kThreads, 0, s>>>((const T*)a, (const T*)b, (T*)y, n);)
  }
  PD_LAUNCH_CHECK("add_kernel");
  return PD_OK;
}
