// C-ABI entry points of the contraction family: plain GEMMs in the three
// transposition forms a Linear layer needs, and the 3x3 / stride 1 / pad 1
// convolution passes on padded-NHWC activations.  bf16 problems run on the
// tcgen05 back end, fp32 problems on the CUDA-core back end; there is no other
// path.
#include "pd_gemm.cuh"

namespace {

int dispatch(const PdGemm& g, cudaStream_t s) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  if (g.dtype == PD_BF16) return pd_gemm_launch_tcgen05(g, s);
  if (g.dtype == PD_F32) return pd_gemm_launch_simt(g, s);
  pd_set_error("gemm: unsupported dtype %d", g.dtype);
  return PD_ERR_INVALID;
}

void init(PdGemm& g) {
  memset(&g, 0, sizeof(g));
  g.num_taps = 1;
  g.num_z = 1;
  g.split_k = 1;
}

// Output mode for fp32 gradient buffers: store when the whole contraction is in
// one CTA and the caller does not accumulate, atomic add otherwise (after
// clearing the destination when the caller does not accumulate).
int prepare_grad_out(PdGemm& g, int accumulate, int64_t rows, int64_t row_elems, cudaStream_t s) {
  if (!accumulate && g.split_k == 1) { g.atomic = 0; return PD_OK; }
  g.atomic = 1;
  if (!accumulate) {
    if (row_elems == g.ldo) {
      PD_CUDA(cudaMemsetAsync(g.out, 0, (size_t)rows * g.ldo * sizeof(float), s));
    } else {
      PD_CUDA(cudaMemset2DAsync(g.out, (size_t)g.ldo * sizeof(float), 0, (size_t)row_elems * sizeof(float), (size_t)rows, s));
    }
  }
  return PD_OK;
}

// Number of K slices for a weight-gradient contraction of `tiles` output tiles and `kblocks` 64-deep K blocks
// on `units` workers (SMs, or SM pairs): the slice count that minimises waves x (K blocks per slice + the cost of
// one atomic epilogue, about six K blocks' worth).
int auto_split(int64_t tiles, int kblocks, int units) {
  if (units < 1) units = 1;
  int best = 1;
  double best_cost = 1e30;
  const int smax = kblocks < 256 ? kblocks : 256;
  for (int s = 1; s <= smax; ++s) {
    const int per = (kblocks + s - 1) / s;
    const int used = (kblocks + per - 1) / per;          // slices that actually get K blocks
    const int64_t waves = (tiles * used + units - 1) / units;
    const double cost = (double)waves * (per + (used > 1 ? 6.0 : 2.0));
    if (cost < best_cost - 1e-9) { best_cost = cost; best = used; }
  }
  return best;
}

// Split for a weight gradient with output [M, N] per z: sized for CTA pairs when the problem qualifies for them.
int grad_split(int dtype, int M, int N, int num_z, int z_per_cta, int bm, int bn, int kblocks) {
  const int sms = pd_num_sms();
  if (dtype == PD_BF16 && pd_gemm_use_pair(M, N, num_z, z_per_cta, 1 << 20)) {
    const int64_t ptiles = (int64_t)((M + 255) / 256) * (N / 256) * num_z;
    const int sp = auto_split(ptiles, kblocks, sms / 2);
    if (pd_gemm_use_pair(M, N, num_z, z_per_cta, sp)) return sp;
  }
  const int64_t tiles = (int64_t)((num_z + z_per_cta - 1) / z_per_cta) * ((M + bm - 1) / bm) * ((N + bn - 1) / bn);
  return auto_split(tiles, kblocks, sms);
}

}  // namespace

// out[M,N] = a[M,K] . b[N,K]^T (+ bias[N]) (ReLU)            -- Linear forward
// pad_hp/pad_wp > 0: rows are padded-NHWC pixels of an (pad_hp x pad_wp) image and border rows are
// written as zero (the first convolution runs as a GEMM over an im2col patch matrix).
PD_EXPORT int pd_gemm_nt(int dtype, const void* a, int64_t lda, const void* b, int64_t ldb, void* out,
                         int out_dtype, int64_t ldo, int M, int N, int K, const void* bias,
                         int bias_dtype, int relu, int pad_hp, int pad_wp, void* stream) {
  PD_REQUIRE(a && b && out, "pd_gemm_nt: null pointer");
  PdGemm g; init(g);
  g.dtype = dtype;
  g.a = a; g.a_rows = M; g.a_cols = K; g.lda = lda; g.a_major = 0;
  g.b = b; g.b_rows = N; g.b_cols = K; g.ldb = ldb; g.b_major = 0;
  g.M = M; g.N = N; g.K = K;
  g.out = out; g.out_dtype = out_dtype; g.ldo = ldo;
  g.bias = bias; g.bias_dtype = bias_dtype; g.relu = relu;
  g.pad_hp = pad_hp; g.pad_wp = pad_wp;
  return dispatch(g, (cudaStream_t)stream);
}

namespace {
// out[m][n] = act(acc[m][n] + bias[n]) as bf16 (or fp32): the second half of a split-K forward contraction.
template <typename O>
__global__ void __launch_bounds__(256)
splitk_finish_kernel(const float* __restrict__ acc, int M, int N, const void* __restrict__ bias, int bias_dtype,
                     int relu, O* __restrict__ out, long long ldo) {
  const long long total = (long long)M * N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(i % N);
    const long long m = i / N;
    float v = acc[i];
    if (bias != nullptr)
      v += bias_dtype == PD_BF16 ? __bfloat162float(((const __nv_bfloat16*)bias)[n]) : ((const float*)bias)[n];
    if (relu) v = fmaxf(v, 0.f);
    out[m * ldo + n] = pd_from_float<O>(v);
  }
}
}  // namespace

// The same product for a short, wide problem - a Linear layer at a batch of 64: [64, 25088] x [4096, 25088]^T has 16
// output tiles for 148 SMs and 205 MB of weights to stream.  The contraction is cut into K slices that add their
// parts into `workspace` (M x N floats, cleared here) with fp32 atomics, and a second small kernel applies bias and
// ReLU and writes `out`.  The order of the additions varies from run to run (last-bit differences).
PD_EXPORT int64_t pd_gemm_nt_splitk_workspace_bytes(int M, int N) { return (int64_t)M * N * (int64_t)sizeof(float); }

PD_EXPORT int pd_gemm_nt_splitk(int dtype, const void* a, int64_t lda, const void* b, int64_t ldb, void* out,
                                int out_dtype, int64_t ldo, int M, int N, int K, const void* bias,
                                int bias_dtype, int relu, void* workspace, int64_t workspace_bytes, void* stream) {
  PD_REQUIRE(a && b && out && workspace, "pd_gemm_nt_splitk: null pointer");
  PD_REQUIRE(dtype == PD_BF16, "pd_gemm_nt_splitk: bf16 operands only");
  PD_REQUIRE(out_dtype == PD_BF16 || out_dtype == PD_F32, "pd_gemm_nt_splitk: bad output type");
  PD_REQUIRE(workspace_bytes >= pd_gemm_nt_splitk_workspace_bytes(M, N), "pd_gemm_nt_splitk: workspace too small");
  cudaStream_t s = (cudaStream_t)stream;
  PdGemm g; init(g);
  g.dtype = dtype;
  g.a = a; g.a_rows = M; g.a_cols = K; g.lda = lda; g.a_major = 0;
  g.b = b; g.b_rows = N; g.b_cols = K; g.ldb = ldb; g.b_major = 0;
  g.M = M; g.N = N; g.K = K;
  g.out = workspace; g.out_dtype = PD_F32; g.ldo = N;
  const int bn = N > 128 ? 256 : (N > 64 ? 128 : 64);
  g.split_k = grad_split(dtype, M, N, 1, 1, 128, bn, (K + 63) / 64);
  int rc = prepare_grad_out(g, 0, M, N, s);
  if (rc != PD_OK) return rc;
  rc = dispatch(g, s);
  if (rc != PD_OK) return rc;
  const long long total = (long long)M * N;
  int grid = (int)((total + 255) / 256);
  if (grid > pd_num_sms() * 8) grid = pd_num_sms() * 8;
  if (out_dtype == PD_BF16)
    splitk_finish_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const float*)workspace, M, N, bias, bias_dtype, relu,
                                                            (__nv_bfloat16*)out, ldo);
  else
    splitk_finish_kernel<float><<<grid, 256, 0, s>>>((const float*)workspace, M, N, bias, bias_dtype, relu, (float*)out, ldo);
  PD_LAUNCH_CHECK("splitk_finish_kernel");
  return PD_OK;
}

// out[M,N] = a[M,K] . b[K,N]; optional mask: out = aux > 0 ? out : 0   -- Linear data gradient
PD_EXPORT int pd_gemm_nn(int dtype, const void* a, int64_t lda, const void* b, int64_t ldb, void* out,
                         int out_dtype, int64_t ldo, int M, int N, int K, const void* relu_aux,
                         int64_t ld_aux, void* stream) {
  PD_REQUIRE(a && b && out, "pd_gemm_nn: null pointer");
  PdGemm g; init(g);
  g.dtype = dtype;
  g.a = a; g.a_rows = M; g.a_cols = K; g.lda = lda; g.a_major = 0;
  g.b = b; g.b_rows = K; g.b_cols = N; g.ldb = ldb; g.b_major = 1;
  g.M = M; g.N = N; g.K = K;
  g.out = out; g.out_dtype = out_dtype; g.ldo = ldo;
  g.relu_aux = relu_aux; g.ld_aux = ld_aux;
  return dispatch(g, (cudaStream_t)stream);
}

// out[M,N] (fp32) (+)= a[K,M]^T . b[K,N]                       -- Linear weight gradient
PD_EXPORT int pd_gemm_tn(int dtype, const void* a, int64_t lda, const void* b, int64_t ldb, float* out,
                         int64_t ldo, int M, int N, int K, int accumulate, int split_k, void* stream) {
  PD_REQUIRE(a && b && out, "pd_gemm_tn: null pointer");
  PdGemm g; init(g);
  g.dtype = dtype;
  g.a = a; g.a_rows = K; g.a_cols = M; g.lda = lda; g.a_major = 1;
  g.b = b; g.b_rows = K; g.b_cols = N; g.ldb = ldb; g.b_major = 1;
  g.M = M; g.N = N; g.K = K;
  g.out = out; g.out_dtype = PD_F32; g.ldo = ldo;
  const int bn = dtype == PD_BF16 ? (N > 128 ? 256 : (N > 64 ? 128 : 64)) : 64;
  const int bm = dtype == PD_BF16 ? 128 : 64;
  g.split_k = split_k > 0 ? split_k : grad_split(dtype, M, N, 1, 1, bm, bn, (K + 63) / 64);
  int rc = prepare_grad_out(g, accumulate, M, N, (cudaStream_t)stream);
  if (rc != PD_OK) return rc;
  return dispatch(g, (cudaStream_t)stream);
}

namespace {
void conv_taps(int Wp, int* shift) {
  for (int r = 0; r < 3; ++r)
    for (int s = 0; s < 3; ++s) shift[r * 3 + s] = (r - 1) * Wp + (s - 1);
}
}  // namespace

// y_pad[P,Cout] = conv3x3(x_pad[P,Cin], w[Cout, 9*Cin]) (+bias) (ReLU); P = N*(H+2)*(W+2).
// w holds the filter as [Cout][r][s][Cin] (the channels-last order of a [Cout,Cin,3,3] tensor).
PD_EXPORT int pd_conv2d_fwd(int dtype, const void* x_pad, int N, int H, int W, int Cin, const void* w,
                            int64_t ldw, int Cout, const void* bias, int bias_dtype, int relu,
                            void* y_pad, void* stream) {
  PD_REQUIRE(x_pad && w && y_pad && N > 0 && H > 0 && W > 0 && Cin > 0 && Cout > 0, "pd_conv2d_fwd: bad arguments");
  const int Hp = H + 2, Wp = W + 2;
  const int64_t P = (int64_t)N * Hp * Wp;
  PD_REQUIRE(P < (1ll << 31), "pd_conv2d_fwd: too many pixels");
  PdGemm g; init(g);
  g.dtype = dtype;
  g.a = x_pad; g.a_rows = P; g.a_cols = Cin; g.lda = Cin; g.a_major = 0;
  g.b = w; g.b_rows = Cout; g.b_cols = 9ll * Cin; g.ldb = ldw; g.b_major = 0;
  g.M = (int)P; g.N = Cout; g.K = Cin;
  g.num_taps = 9;
  int shift[9]; conv_taps(Wp, shift);
  for (int t = 0; t < 9; ++t) { g.a_tap_row[t] = shift[t]; g.b_tap_col[t] = t * Cin; }
  g.share_tap_rows = 1;
  g.out = y_pad; g.out_dtype = dtype; g.ldo = Cout;
  g.bias = bias; g.bias_dtype = bias_dtype; g.relu = relu;
  g.pad_hp = Hp; g.pad_wp = Wp;
  return dispatch(g, (cudaStream_t)stream);
}

// dx_pad[P,Cin] = sum_t dy_pad[p - shift_t, :] . w[:, t, :]; optional ReLU mask by x_pad (> 0).
PD_EXPORT int pd_conv2d_dgrad(int dtype, const void* dy_pad, int N, int H, int W, int Cout, const void* w,
                              int64_t ldw, int Cin, const void* relu_aux, void* dx_pad, void* stream) {
  PD_REQUIRE(dy_pad && w && dx_pad && N > 0 && H > 0 && W > 0 && Cin > 0 && Cout > 0, "pd_conv2d_dgrad: bad arguments");
  const int Hp = H + 2, Wp = W + 2;
  const int64_t P = (int64_t)N * Hp * Wp;
  PD_REQUIRE(P < (1ll << 31), "pd_conv2d_dgrad: too many pixels");
  PdGemm g; init(g);
  g.dtype = dtype;
  g.a = dy_pad; g.a_rows = P; g.a_cols = Cout; g.lda = Cout; g.a_major = 0;
  g.b = w; g.b_rows = Cout; g.b_cols = 9ll * Cin; g.ldb = ldw; g.b_major = 1;
  g.M = (int)P; g.N = Cin; g.K = Cout;
  g.num_taps = 9;
  int shift[9]; conv_taps(Wp, shift);
  for (int t = 0; t < 9; ++t) { g.a_tap_row[t] = -shift[t]; g.b_tap_col[t] = t * Cin; }
  g.share_tap_rows = 1;
  g.out = dx_pad; g.out_dtype = dtype; g.ldo = Cin;
  g.pad_hp = Hp; g.pad_wp = Wp;
  g.relu_aux = relu_aux; g.ld_aux = Cin;
  return dispatch(g, (cudaStream_t)stream);
}

// dw[Cout, 9*Cin] (fp32, leading dim lddw) (+)= sum_p dy_pad[p, co] * x_pad[p + shift_t, ci]
PD_EXPORT int pd_conv2d_wgrad(int dtype, const void* x_pad, const void* dy_pad, int N, int H, int W,
                              int Cin, int Cout, float* dw, int64_t lddw, int accumulate, int split_k,
                              void* stream) {
  PD_REQUIRE(x_pad && dy_pad && dw && N > 0 && H > 0 && W > 0 && Cin > 0 && Cout > 0, "pd_conv2d_wgrad: bad arguments");
  const int Hp = H + 2, Wp = W + 2;
  const int64_t P = (int64_t)N * Hp * Wp;
  PD_REQUIRE(P < (1ll << 31), "pd_conv2d_wgrad: too many pixels");
  PdGemm g; init(g);
  g.dtype = dtype;
  g.a = dy_pad; g.a_rows = P; g.a_cols = Cout; g.lda = Cout; g.a_major = 1;
  g.b = x_pad; g.b_rows = P; g.b_cols = Cin; g.ldb = Cin; g.b_major = 1;
  g.M = Cout; g.N = Cin; g.K = (int)P;
  g.num_z = 9;
  int shift[9]; conv_taps(Wp, shift);
  for (int t = 0; t < 9; ++t) g.z_b_row[t] = shift[t];
  g.z_out_col = Cin;
  g.z_group = 4;
  g.out = dw; g.out_dtype = PD_F32; g.ldo = lddw;
  const int bn = dtype == PD_BF16 ? (Cin > 128 ? 256 : (Cin > 64 ? 128 : 64)) : 64;
  const int bm = dtype == PD_BF16 ? 128 : 64;
  // bf16: up to 256 accumulator columns per CTA, i.e. several taps share one CTA (z groups)
  const int per_cta = dtype == PD_BF16 ? (256 / bn < 4 ? (256 / bn < 1 ? 1 : 256 / bn) : 4) : 1;
  g.split_k = split_k > 0 ? split_k : grad_split(dtype, Cout, Cin, 9, per_cta, bm, bn, (int)((P + 63) / 64));
  int rc = prepare_grad_out(g, accumulate, Cout, 9ll * Cin, (cudaStream_t)stream);
  if (rc != PD_OK) return rc;
  return dispatch(g, (cudaStream_t)stream);
}
