// fp32 contraction back end (CUDA cores).  Same problem description as the
// tcgen05 path; used for the fp32 parity configuration, where tensor-core input
// rounding would not meet the 1e-3 tolerance after 20 training steps.
#include "pd_gemm.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, kThreads = 256;

struct SParams {
  const float* a; long long a_rows, lda; int a_major;
  const float* b; long long b_rows, ldb; int b_major;
  int M, N, K, num_taps;
  int a_row0, a_col0, b_row0, b_col0;
  int a_tap_row[PD_MAX_TAPS], a_tap_col[PD_MAX_TAPS];
  int b_tap_row[PD_MAX_TAPS], b_tap_col[PD_MAX_TAPS];
  int z_b_row[PD_MAX_TAPS]; long long z_out_col;
  int split_k, k_per_split;
  float* out; long long ldo; int atomic;
  const float* bias; int relu; int pad_hp, pad_wp;
  const float* relu_aux; long long ld_aux;
};

__global__ void __launch_bounds__(kThreads)
gemm_simt_kernel(const SParams p) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int z = blockIdx.z / p.split_k, split = blockIdx.z % p.split_k;
  const int k_begin = split * p.k_per_split;
  const int k_end = min(p.K, k_begin + p.k_per_split);
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;   // 16 x 16 threads, 4x4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int t = 0; t < p.num_taps; ++t) {
    for (int k0 = k_begin; k0 < k_end; k0 += BK) {
      // A tile
      if (p.a_major == 0) {
        // thread -> (row = tid / 4, k = (tid % 4) * 4 .. +3): k contiguous in memory
        const int row = threadIdx.x >> 2, kq = (threadIdx.x & 3) << 2;
        const long long gr = (long long)p.a_row0 + m0 + row + p.a_tap_row[t];
        const bool rok = (m0 + row < p.M) && gr >= 0 && gr < p.a_rows;
        const float* src = p.a + gr * p.lda + p.a_col0 + p.a_tap_col[t];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k = k0 + kq + j;
          As[kq + j][row] = (rok && k < k_end) ? src[k] : 0.f;
        }
      } else {
        // thread -> (k = tid / 16, m = (tid % 16) * 4 .. +3): m contiguous in memory
        const int kk = threadIdx.x >> 4, mq = (threadIdx.x & 15) << 2;
        const int k = k0 + kk;
        const long long gr = (long long)p.a_row0 + k + p.a_tap_row[t];
        const bool rok = k < k_end && gr >= 0 && gr < p.a_rows;
        const float* src = p.a + gr * p.lda + p.a_col0 + p.a_tap_col[t] + m0;
#pragma unroll
        for (int j = 0; j < 4; ++j) As[kk][mq + j] = (rok && m0 + mq + j < p.M) ? src[mq + j] : 0.f;
      }
      // B tile
      if (p.b_major == 0) {
        const int row = threadIdx.x >> 2, kq = (threadIdx.x & 3) << 2;
        const long long gr = (long long)p.b_row0 + n0 + row + p.b_tap_row[t] + p.z_b_row[z];
        const bool rok = (n0 + row < p.N) && gr >= 0 && gr < p.b_rows;
        const float* src = p.b + gr * p.ldb + p.b_col0 + p.b_tap_col[t];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k = k0 + kq + j;
          Bs[kq + j][row] = (rok && k < k_end) ? src[k] : 0.f;
        }
      } else {
        const int kk = threadIdx.x >> 4, nq = (threadIdx.x & 15) << 2;
        const int k = k0 + kk;
        const long long gr = (long long)p.b_row0 + k + p.b_tap_row[t] + p.z_b_row[z];
        const bool rok = k < k_end && gr >= 0 && gr < p.b_rows;
        const float* src = p.b + gr * p.ldb + p.b_col0 + p.b_tap_col[t] + n0;
#pragma unroll
        for (int j = 0; j < 4; ++j) Bs[kk][nq + j] = (rok && n0 + nq + j < p.N) ? src[nq + j] : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        float av[4], bv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }
      __syncthreads();
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
    bool border = false;
    if (p.pad_wp > 0) {
      const int wp = m % p.pad_wp, hp = (m / p.pad_wp) % p.pad_hp;
      border = wp == 0 || wp == p.pad_wp - 1 || hp == 0 || hp == p.pad_hp - 1;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      float v = acc[i][j];
      if (p.bias) v += p.bias[n];
      if (p.relu) v = fmaxf(v, 0.f);
      if (p.relu_aux && !(p.relu_aux[(long long)m * p.ld_aux + n] > 0.f)) v = 0.f;
      if (border) v = 0.f;
      float* o = p.out + (long long)m * p.ldo + (long long)z * p.z_out_col + n;
      if (p.atomic) atomicAdd(o, v);
      else *o = v;
    }
  }
}

}  // namespace

int pd_gemm_launch_simt(const PdGemm& g, cudaStream_t stream) {
  PD_REQUIRE(g.dtype == PD_F32 && g.out_dtype == PD_F32, "simt gemm: operands and output must be fp32");
  PD_REQUIRE(g.bias == nullptr || g.bias_dtype == PD_F32, "simt gemm: bias must be fp32");
  PD_REQUIRE(g.M > 0 && g.N > 0 && g.K > 0, "simt gemm: empty problem");
  PD_REQUIRE(g.num_taps >= 1 && g.num_taps <= PD_MAX_TAPS && g.num_z >= 1 && g.num_z <= PD_MAX_TAPS, "simt gemm: bad tap/z count");
  PD_REQUIRE(g.split_k >= 1 && (g.split_k == 1 || g.atomic), "simt gemm: split_k needs the atomic epilogue");
  SParams p;
  memset(&p, 0, sizeof(p));
  p.a = (const float*)g.a; p.a_rows = g.a_rows; p.lda = g.lda; p.a_major = g.a_major;
  p.b = (const float*)g.b; p.b_rows = g.b_rows; p.ldb = g.ldb; p.b_major = g.b_major;
  p.M = g.M; p.N = g.N; p.K = g.K; p.num_taps = g.num_taps;
  p.a_row0 = g.a_row0; p.a_col0 = g.a_col0; p.b_row0 = g.b_row0; p.b_col0 = g.b_col0;
  for (int t = 0; t < PD_MAX_TAPS; ++t) {
    p.a_tap_row[t] = g.a_tap_row[t]; p.a_tap_col[t] = g.a_tap_col[t];
    p.b_tap_row[t] = g.b_tap_row[t]; p.b_tap_col[t] = g.b_tap_col[t];
    p.z_b_row[t] = g.z_b_row[t];
  }
  p.z_out_col = g.z_out_col;
  int kblocks = (g.K + BK - 1) / BK;
  int split = g.split_k > kblocks ? kblocks : g.split_k;
  int per = (kblocks + split - 1) / split;
  split = (kblocks + per - 1) / per;
  p.split_k = split; p.k_per_split = per * BK;
  p.out = (float*)g.out; p.ldo = g.ldo; p.atomic = g.atomic;
  p.bias = (const float*)g.bias; p.relu = g.relu; p.pad_hp = g.pad_hp; p.pad_wp = g.pad_wp;
  p.relu_aux = (const float*)g.relu_aux; p.ld_aux = g.ld_aux;
  dim3 grid((g.M + BM - 1) / BM, (g.N + BN - 1) / BN, g.num_z * split);
  PD_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "simt gemm: grid too large");
  gemm_simt_kernel<<<grid, kThreads, 0, stream>>>(p);
  PD_LAUNCH_CHECK("gemm_simt_kernel");
  return PD_OK;
}
