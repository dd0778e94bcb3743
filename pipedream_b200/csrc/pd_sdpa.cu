// Causal self-attention of the transformer stages (softmax(Q K^T / sqrt(d)) V per head), bf16, head size 64,
// sequence length a multiple of 128: five batched contractions on the tensor cores and two row kernels.
//
//   forward   S = Q K^T            [T, T] per (batch, head), only the tiles on and below the diagonal
//             P = softmax(scale S) in place (row kernel, fp32 statistics, zeros above the diagonal)
//             O = P V              contraction over the keys up to the diagonal
//   backward  dP = dO V^T          tiles on and below the diagonal
//             dS = P (dP - rowsum(P dP)) scale   in place (row kernel)
//             dV = P^T dO,  dK = dS^T Q          contraction over the queries from the diagonal on
//             dQ = dS K                          contraction over the keys up to the diagonal
//
// Q, K and V are read in place from the fused projection's output [B, T, 3, H, 64] and the three gradients are
// written in place into a tensor of the same shape, so nothing is transposed or copied.  P is kept for the backward
// pass (B H T^2 bf16); the scores round to bf16 between the contraction and the softmax.
//
// The batched contraction is a small relative of the big persistent kernel: one 128 x 128 (or 128 x 64) tile per
// CTA, blockIdx.y / .z = head / batch, a three-stage TMA ring, one issuing thread, four epilogue warps.  Operands
// are taken K-major or MN-major as they lie (descriptor flags), which gives the three transposition forms:
//   NT: A [M, K] . B [N, K]^T     NN: A [M, K] . B [K, N]     TN: A [K, M]^T . B [K, N]
#include <cstring>
#include <mutex>

#include "pd_gemm.cuh"
#include "pd_sm100_ptx.cuh"

namespace {

using namespace pd_sm100;

constexpr int kThreads = 192;          // warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: epilogue
constexpr int kStages = 3;
constexpr int kHead = 64;              // head size this file is written for
constexpr uint32_t kTileA = 128 * kBlockK * 2;          // 16 KiB

struct Coord { int row_b, row_h, col_h; };              // TMA coordinate offsets per batch / head index

struct BgemmP {
  int K;                    // contraction length per (batch, head), a multiple of 64
  int n_tiles;              // tiles along N
  int block_n;              // 128 or 64
  int causal;               // 0: none; 1: skip tiles right of the diagonal (n0 > m0 + 127);
                            // 2: contract k < m0 + 128 only; 3: contract k >= m0 only
  Coord a, b;
  __nv_bfloat16* out;
  long long out_b, out_h, ldo;   // elements
  int* err;
  uint32_t idesc;
};

template <int FORM>         // 0: NT, 1: NN, 2: TN
__global__ void __launch_bounds__(kThreads, 1)
attn_bgemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const BgemmP p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_holder;

  const int m0 = (int)(blockIdx.x / p.n_tiles) * 128;
  const int n0 = (int)(blockIdx.x % p.n_tiles) * p.block_n;
  if (p.causal == 1 && n0 > m0 + 127) return;            // the whole CTA: nothing allocated yet
  const int h = blockIdx.y, b = blockIdx.z;
  int kb0 = 0, kb1 = p.K / kBlockK;
  if (p.causal == 2) kb1 = min(kb1, (m0 + 128) / kBlockK);
  if (p.causal == 3) kb0 = m0 / kBlockK;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t b_bytes = (uint32_t)p.block_n * kBlockK * 2;
  const uint32_t stage_bytes = kTileA + b_bytes;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&acc_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_holder)), "r"(128u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = tmem_base_holder;

  if (warp == 0) {
    if (lane == 0) {
      const int ar = p.a.row_b * b + p.a.row_h * h, ac = p.a.col_h * h;
      const int br = p.b.row_b * b + p.b.row_h * h, bc = p.b.col_h * h;
      uint32_t it = 0;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = (int)(it % kStages);
        const uint32_t ph = (it / kStages) & 1u;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, p.err, 11)) break;
        const uint32_t fb = smem_u32(&full_bar[s]);
        const uint32_t sa = smem0 + (uint32_t)s * stage_bytes, sb = sa + kTileA;
        mbar_expect_tx(fb, stage_bytes);
        if (FORM == 2) {            // A stored [K, M]: two 64-wide atoms of 64 K rows
          tma_load_2d(sa, &map_a, fb, ac + m0, ar + kb * kBlockK);
          tma_load_2d(sa + kAtomBytes, &map_a, fb, ac + m0 + 64, ar + kb * kBlockK);
        } else {                    // A stored [M, K]
          tma_load_2d(sa, &map_a, fb, ac + kb * kBlockK, ar + m0);
        }
        if (FORM == 0) {            // B stored [N, K]
          tma_load_2d(sb, &map_b, fb, bc + kb * kBlockK, br + n0);
        } else {                    // B stored [K, N]: 64-wide atoms
          for (int j = 0; j < p.block_n / 64; ++j)
            tma_load_2d(sb + (uint32_t)j * kAtomBytes, &map_b, fb, bc + n0 + j * 64, br + kb * kBlockK);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr int a_mn = FORM == 2 ? 1 : 0, b_mn = FORM == 0 ? 0 : 1;
      const uint32_t adv_a = a_mn ? (16u * 128u) >> 4 : (16u * 2u) >> 4;
      const uint32_t adv_b = b_mn ? (16u * 128u) >> 4 : (16u * 2u) >> 4;
      bool ok = true;
      uint32_t it = 0;
      for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
        const int s = (int)(it % kStages);
        const uint32_t ph = (it / kStages) & 1u;
        ok = mbar_wait(smem_u32(&full_bar[s]), ph, p.err, 12);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = smem0 + (uint32_t)s * stage_bytes;
        const uint64_t da = make_desc(sa, a_mn), db = make_desc(sa + kTileA, b_mn);
        const uint32_t a_lo = (uint32_t)da, a_hi = (uint32_t)(da >> 32), b_lo = (uint32_t)db, b_hi = (uint32_t)(db >> 32);
#pragma unroll
        for (int kk = 0; kk < kBlockK / 16; ++kk)
          umma_lo<1, 2>(tmem_acc, a_lo + kk * adv_a, a_hi, b_lo + kk * adv_b, b_hi, p.idesc, (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(smem_u32(&empty_bar[s]));
      }
      if (ok) umma_commit(smem_u32(&acc_bar));
    }
  } else {
    const int lg = warp & 3;
    const int m = m0 + lg * 32 + lane;
    // (a tile with an empty contraction range cannot occur: the diagonal block is always inside it)
    bool ok = mbar_wait(smem_u32(&acc_bar), 0, p.err, 13);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      __nv_bfloat16* o = p.out + (long long)b * p.out_b + (long long)h * p.out_h + (long long)m * p.ldo + n0;
      for (int cc = 0; cc < p.block_n; cc += 32) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tmem_acc + ((uint32_t)(lg * 32) << 16) + (uint32_t)cc, r);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
          w[e] = *reinterpret_cast<uint32_t*>(&v);
        }
        // 32-byte stores: a lane writes whole sectors of its row (rows, leading dimensions and tile origins are
        // multiples of 64 bytes here)
#pragma unroll
        for (int q = 0; q < 2; ++q)
          asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                       ::"l"(o + cc + q * 16), "r"(w[q * 8]), "r"(w[q * 8 + 1]), "r"(w[q * 8 + 2]), "r"(w[q * 8 + 3]),
                         "r"(w[q * 8 + 4]), "r"(w[q * 8 + 5]), "r"(w[q * 8 + 6]), "r"(w[q * 8 + 7])
                       : "memory");
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(128u) : "memory");
  }
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
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int kMaxVecPerLane = 8;      // T <= 32 * 8 * 8 = 2048
// (the row kernels are instantiated for 1, 2, 4 and 8 vectors of 8 per lane - T up to 256, 512, 1024, 2048 - so that
// a row of 512 keeps 16 values per lane in registers, not 64, and enough warps fit on an SM to hide the latency)

// One warp per row of the [B H T, T] score matrix, in place: P[i, j] = softmax_j(scale S[i, j]) over j <= i, 0 beyond
// (the tiles right of the diagonal were never written by the contraction: every element there is written here).
template <int VPL>
__global__ void __launch_bounds__(256)
causal_softmax_fwd_kernel(__nv_bfloat16* __restrict__ s, int64_t rows, int T, float scale) {
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int t = (int)(row % T);
  uint4* base = reinterpret_cast<uint4*>(s + row * T);
  const int nvec = T / 8;
  float v[VPL][8];
  float mx = -3.0e38f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec && vi * 8 <= t) {
      unpack8(base[vi], v[i]);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        v[i][k] = (vi * 8 + k <= t) ? v[i][k] * scale : -3.0e38f;
        mx = fmaxf(mx, v[i][k]);
      }
    }
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec && vi * 8 <= t) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        v[i][k] = (vi * 8 + k <= t) ? __expf(v[i][k] - mx) : 0.f;
        sum += v[i][k];
      }
    }
  }
  const float inv = 1.f / warp_sum(sum);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = (vi * 8 <= t) ? v[i][k] * inv : 0.f;
      base[vi] = pack8(o);
    }
  }
}

// dS[i, j] = P[i, j] (dP[i, j] - sum_k P[i, k] dP[i, k]) scale over j <= i, 0 beyond; in place on dP.
template <int VPL>
__global__ void __launch_bounds__(256)
causal_softmax_bwd_kernel(const __nv_bfloat16* __restrict__ p, __nv_bfloat16* __restrict__ dp, int64_t rows, int T,
                          float scale) {
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int t = (int)(row % T);
  const uint4* pb = reinterpret_cast<const uint4*>(p + row * T);
  uint4* db = reinterpret_cast<uint4*>(dp + row * T);
  const int nvec = T / 8;
  float pv[VPL][8], dv[VPL][8];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec && vi * 8 <= t) {
      unpack8(pb[vi], pv[i]);
      unpack8(db[vi], dv[i]);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (vi * 8 + k <= t) dot = fmaf(pv[i][k], dv[i][k], dot);
    }
  }
  dot = warp_sum(dot);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        o[k] = (vi * 8 <= t && vi * 8 + k <= t) ? pv[i][k] * (dv[i][k] - dot) * scale : 0.f;
      db[vi] = pack8(o);
    }
  }
}

std::mutex g_attr_mu;
bool g_attr_set[64];

struct Operand { const void* base; int64_t rows, cols, ld; Coord c; };

int launch_bgemm(int form, const Operand& a, const Operand& b, int M, int N, int K, int block_n, int causal,
                 __nv_bfloat16* out, long long out_b, long long out_h, long long ldo, int B, int H, cudaStream_t s) {
  BgemmP p;
  memset(&p, 0, sizeof(p));
  p.K = K; p.block_n = block_n; p.n_tiles = N / block_n; p.causal = causal;
  p.a = a.c; p.b = b.c;
  p.out = out; p.out_b = out_b; p.out_h = out_h; p.ldo = ldo;
  const int a_mn = form == 2 ? 1 : 0, b_mn = form == 0 ? 0 : 1;
  p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
            ((uint32_t)(block_n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  int rc = pd_gemm_error_word(&p.err);
  if (rc != PD_OK) return rc;
  CUtensorMap ma, mb;
  rc = pd_make_map_2d(&ma, a.base, a.rows, a.cols, a.ld, 64, form == 2 ? kBlockK : 128);
  if (rc != PD_OK) return rc;
  rc = pd_make_map_2d(&mb, b.base, b.rows, b.cols, b.ld, 64, form == 0 ? block_n : kBlockK);
  if (rc != PD_OK) return rc;
  const size_t smem = (size_t)kStages * (kTileA + (size_t)block_n * kBlockK * 2) + 1024;
  {
    int dev = 0;
    PD_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_attr_mu);
    if (dev >= 0 && dev < 64 && !g_attr_set[dev]) {
      PD_CUDA(cudaFuncSetAttribute(attn_bgemm_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
      PD_CUDA(cudaFuncSetAttribute(attn_bgemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
      PD_CUDA(cudaFuncSetAttribute(attn_bgemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
      g_attr_set[dev] = true;
    }
  }
  const dim3 grid((unsigned)((M / 128) * p.n_tiles), (unsigned)H, (unsigned)B);
  if (form == 0) attn_bgemm_kernel<0><<<grid, kThreads, smem, s>>>(ma, mb, p);
  else if (form == 1) attn_bgemm_kernel<1><<<grid, kThreads, smem, s>>>(ma, mb, p);
  else attn_bgemm_kernel<2><<<grid, kThreads, smem, s>>>(ma, mb, p);
  PD_LAUNCH_CHECK("attn_bgemm_kernel");
  return PD_OK;
}

int check_shape(const char* who, int dtype, int B, int T, int H, int d) {
  if (dtype != PD_BF16) { pd_set_error("%s: bf16 only", who); return PD_ERR_INVALID; }
  if (B < 1 || H < 1 || d != kHead || T < 128 || (T % 128) != 0 || T > 32 * 8 * kMaxVecPerLane) {
    pd_set_error("%s: needs head size 64 and a sequence length that is a multiple of 128 (at most 2048), got T=%d d=%d", who, T, d);
    return PD_ERR_INVALID;
  }
  if ((int64_t)B * H * T >= (1ll << 31) || (int64_t)B * T >= (1ll << 31)) { pd_set_error("%s: too many rows", who); return PD_ERR_INVALID; }
  return PD_OK;
}

}  // namespace

// out [B, T, H*64] = causal attention of qkv [B, T, 3, H, 64] (q, k, v of one fused projection); probs [B*H, T, T]
// receives the attention weights (kept for pd_sdpa_causal_bwd).
PD_EXPORT int pd_sdpa_causal_fwd(int dtype, const void* qkv, int B, int T, int H, int d, float scale, void* out,
                                 void* probs, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(qkv && out && probs, "pd_sdpa_causal_fwd: null pointer");
  rc = check_shape("pd_sdpa_causal_fwd", dtype, B, T, H, d);
  if (rc != PD_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const int C = H * d;
  const __nv_bfloat16* base = (const __nv_bfloat16*)qkv;
  const int64_t BT = (int64_t)B * T, BHT = (int64_t)B * H * T;
  const Operand q = {base, BT, C, 3ll * C, {T, 0, d}};
  const Operand k = {base + C, BT, C, 3ll * C, {T, 0, d}};
  const Operand v = {base + 2 * C, BT, C, 3ll * C, {T, 0, d}};
  const Operand pr = {probs, BHT, T, T, {H * T, T, 0}};
  // S = Q K^T
  rc = launch_bgemm(0, q, k, T, T, d, 128, 1, (__nv_bfloat16*)probs, (long long)H * T * T, (long long)T * T, T, B, H, s);
  if (rc != PD_OK) return rc;
  const unsigned sgrid = (unsigned)((BHT + 7) / 8);
  if (T <= 256) causal_softmax_fwd_kernel<1><<<sgrid, 256, 0, s>>>((__nv_bfloat16*)probs, BHT, T, scale);
  else if (T <= 512) causal_softmax_fwd_kernel<2><<<sgrid, 256, 0, s>>>((__nv_bfloat16*)probs, BHT, T, scale);
  else if (T <= 1024) causal_softmax_fwd_kernel<4><<<sgrid, 256, 0, s>>>((__nv_bfloat16*)probs, BHT, T, scale);
  else causal_softmax_fwd_kernel<8><<<sgrid, 256, 0, s>>>((__nv_bfloat16*)probs, BHT, T, scale);
  PD_LAUNCH_CHECK("causal_softmax_fwd_kernel");
  // O = P V
  return launch_bgemm(1, pr, v, T, d, T, 64, 2, (__nv_bfloat16*)out, (long long)T * C, d, C, B, H, s);
}

// dqkv [B, T, 3, H, 64] from dout [B, T, H*64]; dscores [B*H, T, T] is scratch.
PD_EXPORT int pd_sdpa_causal_bwd(int dtype, const void* qkv, const void* probs, const void* dout, int B, int T, int H,
                                 int d, float scale, void* dqkv, void* dscores, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(qkv && probs && dout && dqkv && dscores, "pd_sdpa_causal_bwd: null pointer");
  rc = check_shape("pd_sdpa_causal_bwd", dtype, B, T, H, d);
  if (rc != PD_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const int C = H * d;
  const __nv_bfloat16* base = (const __nv_bfloat16*)qkv;
  __nv_bfloat16* g = (__nv_bfloat16*)dqkv;
  const int64_t BT = (int64_t)B * T, BHT = (int64_t)B * H * T;
  const Operand q = {base, BT, C, 3ll * C, {T, 0, d}};
  const Operand k = {base + C, BT, C, 3ll * C, {T, 0, d}};
  const Operand v = {base + 2 * C, BT, C, 3ll * C, {T, 0, d}};
  const Operand dO = {dout, BT, C, C, {T, 0, d}};
  const Operand pr = {probs, BHT, T, T, {H * T, T, 0}};
  const Operand ds = {dscores, BHT, T, T, {H * T, T, 0}};
  const long long gb = (long long)T * 3 * C, gh = d, gld = 3ll * C;
  // dP = dO V^T
  rc = launch_bgemm(0, dO, v, T, T, d, 128, 1, (__nv_bfloat16*)dscores, (long long)H * T * T, (long long)T * T, T, B, H, s);
  if (rc != PD_OK) return rc;
  // dV = P^T dO (before dP is overwritten by dS: P is read, dP not)
  rc = launch_bgemm(2, pr, dO, T, d, T, 64, 3, g + 2 * C, gb, gh, gld, B, H, s);
  if (rc != PD_OK) return rc;
  const unsigned sgrid = (unsigned)((BHT + 7) / 8);
  const __nv_bfloat16* pp = (const __nv_bfloat16*)probs;
  __nv_bfloat16* dd = (__nv_bfloat16*)dscores;
  if (T <= 256) causal_softmax_bwd_kernel<1><<<sgrid, 256, 0, s>>>(pp, dd, BHT, T, scale);
  else if (T <= 512) causal_softmax_bwd_kernel<2><<<sgrid, 256, 0, s>>>(pp, dd, BHT, T, scale);
  else if (T <= 1024) causal_softmax_bwd_kernel<4><<<sgrid, 256, 0, s>>>(pp, dd, BHT, T, scale);
  else causal_softmax_bwd_kernel<8><<<sgrid, 256, 0, s>>>(pp, dd, BHT, T, scale);
  PD_LAUNCH_CHECK("causal_softmax_bwd_kernel");
  // dK = dS^T Q, dQ = dS K
  rc = launch_bgemm(2, ds, q, T, d, T, 64, 3, g + C, gb, gh, gld, B, H, s);
  if (rc != PD_OK) return rc;
  return launch_bgemm(1, ds, k, T, d, T, 64, 2, g, gb, gh, gld, B, H, s);
}
