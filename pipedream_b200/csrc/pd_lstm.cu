// Single-layer unidirectional LSTM over [T, B, *] sequences (torch.nn.LSTM(I, H) as used by the
// translation stages, runtime/translation/models/gnmt_large/gpus=4/stage0.py:11-19): the time loop.
//
// The input projection x_t . W_ih^T (+ b_ih) for all time steps is one large contraction done by the
// caller (pd_gemm_nt).  These entry points run the recurrence: per step one contraction with W_hh on
// the tensor cores (bf16; CUDA cores for fp32) and one fused cell kernel (gate activations, cell and
// hidden update, all statistics in fp32).  For bf16 with B <= 128 and H <= 1184 the forward recurrence runs
// instead as one cooperative kernel for the whole sequence (pd_lstm_persist.cu).  The whole loop is enqueued from C++ so that a layer costs
// one call from the host language, not two per time step.  Gate order is torch's: i, f, g, o.
#include "pd_gemm.cuh"
#include <cstdlib>

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// gates = gx + gh (+ b_hh); i,f,o = sigmoid, g = tanh; c = f*c_prev + i*g; h = o*tanh(c).
template <typename T>
__global__ void __launch_bounds__(kThreads)
lstm_cell_fwd_kernel(const T* __restrict__ gx, const float* __restrict__ gh, const T* __restrict__ b_hh,
                     const float* __restrict__ c_prev, T* __restrict__ act, float* __restrict__ c_out,
                     T* __restrict__ h_out, int B, int H) {
  const int64_t total = (int64_t)B * H;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int b = (int)(i / H), u = (int)(i % H);
    const int64_t base = (int64_t)b * 4 * H + u;
    float g4[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float v = pd_to_float(gx[base + (int64_t)k * H]);
      if (gh != nullptr) v += gh[base + (int64_t)k * H];
      if (b_hh != nullptr) v += pd_to_float(b_hh[u + k * H]);
      g4[k] = v;
    }
    const float ig = sigmoidf_(g4[0]), fg = sigmoidf_(g4[1]), gg = tanhf(g4[2]), og = sigmoidf_(g4[3]);
    const float cp = c_prev != nullptr ? c_prev[i] : 0.f;
    const float c = fg * cp + ig * gg;
    c_out[i] = c;
    h_out[i] = pd_from_float<T>(og * tanhf(c));
    act[base] = pd_from_float<T>(ig);
    act[base + H] = pd_from_float<T>(fg);
    act[base + 2 * (int64_t)H] = pd_from_float<T>(gg);
    act[base + 3 * (int64_t)H] = pd_from_float<T>(og);
  }
}

// dh = dy (+ dh_next); dc (in: from step t+1, out: for step t-1); dgates = pre-activation gradients.
// dh_next is cleared after it is read so that the next split-K contraction can accumulate into it.
template <typename T>
__global__ void __launch_bounds__(kThreads)
lstm_cell_bwd_kernel(const T* __restrict__ dy, float* __restrict__ dh_next, float* __restrict__ dc,
                     const T* __restrict__ act, const float* __restrict__ c_t, const float* __restrict__ c_prev,
                     T* __restrict__ dgates, int B, int H, int first) {
  const int64_t total = (int64_t)B * H;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int b = (int)(i / H), u = (int)(i % H);
    const int64_t base = (int64_t)b * 4 * H + u;
    float dh = dy != nullptr ? pd_to_float(dy[i]) : 0.f;
    if (!first) dh += dh_next[i];
    dh_next[i] = 0.f;
    const float ig = pd_to_float(act[base]), fg = pd_to_float(act[base + H]);
    const float gg = pd_to_float(act[base + 2 * (int64_t)H]), og = pd_to_float(act[base + 3 * (int64_t)H]);
    const float tc = tanhf(c_t[i]);
    float dcv = dh * og * (1.f - tc * tc) + (first ? 0.f : dc[i]);
    const float cp = c_prev != nullptr ? c_prev[i] : 0.f;
    const float d_o = dh * tc;
    const float d_i = dcv * gg, d_f = dcv * cp, d_g = dcv * ig;
    dc[i] = dcv * fg;
    dgates[base] = pd_from_float<T>(d_i * ig * (1.f - ig));
    dgates[base + H] = pd_from_float<T>(d_f * fg * (1.f - fg));
    dgates[base + 2 * (int64_t)H] = pd_from_float<T>(d_g * (1.f - gg * gg));
    dgates[base + 3 * (int64_t)H] = pd_from_float<T>(d_o * og * (1.f - og));
  }
}

int cell_grid(int B, int H) {
  int64_t blocks = ((int64_t)B * H + kThreads - 1) / kThreads;
  int64_t cap = (int64_t)pd_num_sms() * 8;
  return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

void init_gemm(PdGemm& g) {
  memset(&g, 0, sizeof(g));
  g.num_taps = 1; g.num_z = 1; g.split_k = 1;
}

int launch(const PdGemm& g, cudaStream_t s) {
  return g.dtype == PD_BF16 ? pd_gemm_launch_tcgen05(g, s) : pd_gemm_launch_simt(g, s);
}

}  // namespace

// Forward recurrence.  gx: [T,B,4H] input projections (+ b_ih) in `dtype`; w_hh: [4H,H]; b_hh: [4H] or
// NULL; y: [T,B,H] (out); act: [T,B,4H] gate activations (out, saved for backward); c_all: [T,B,H] fp32
// cell states (out, saved); gh_ws: [B,4H] fp32 scratch.  Initial hidden and cell state are zero.
PD_EXPORT int pd_lstm_fwd(int dtype, const void* gx, const void* w_hh, const void* b_hh, int T, int B, int H,
                          void* y, void* act, float* c_all, float* gh_ws, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(gx && w_hh && y && act && c_all && gh_ws && T > 0 && B > 0 && H > 0, "pd_lstm_fwd: bad arguments");
  PD_REQUIRE(dtype == PD_F32 || dtype == PD_BF16, "pd_lstm_fwd: bad dtype");
  PD_REQUIRE(dtype == PD_F32 || (H % 8) == 0, "pd_lstm_fwd: H must be a multiple of 8 for bf16");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PD_BF16) {
    // the whole sequence as one cooperative kernel where it applies (PD_LSTM_PERSISTENT=0 switches it off)
    static const bool enabled = [] { const char* e = getenv("PD_LSTM_PERSISTENT"); return !(e && e[0] == '0'); }();
    if (enabled) {
      const int prc = pd_lstm_fwd_persistent(gx, w_hh, b_hh, T, B, H, y, act, c_all, (unsigned int*)gh_ws, s);
      if (prc != 1) return prc;
    }
  }
  const int es = pd_elem_size(dtype);
  const int64_t BH = (int64_t)B * H;
  const int grid = cell_grid(B, H);
  for (int t = 0; t < T; ++t) {
    const char* gx_t = (const char*)gx + (int64_t)t * 4 * BH * es;
    char* y_t = (char*)y + (int64_t)t * BH * es;
    char* act_t = (char*)act + (int64_t)t * 4 * BH * es;
    float* c_t = c_all + (int64_t)t * BH;
    const float* gh = nullptr;
    if (t > 0) {
      PdGemm g; init_gemm(g);
      g.dtype = dtype;
      // whole-sequence map, step selected by the row origin (fp32 path: plain pointer arithmetic inside)
      g.a = y; g.a_rows = (int64_t)T * B; g.a_cols = H; g.lda = H; g.a_major = 0;
      g.a_row0 = (t - 1) * B;
      g.b = w_hh; g.b_rows = 4 * H; g.b_cols = H; g.ldb = H; g.b_major = 0;
      g.M = B; g.N = 4 * H; g.K = H;
      g.out = gh_ws; g.out_dtype = PD_F32; g.ldo = 4 * H;
      rc = launch(g, s);
      if (rc != PD_OK) return rc;
      gh = gh_ws;
    }
    const float* c_prev = t > 0 ? c_all + (int64_t)(t - 1) * BH : nullptr;
    if (dtype == PD_F32)
      lstm_cell_fwd_kernel<float><<<grid, kThreads, 0, s>>>((const float*)gx_t, gh, (const float*)b_hh, c_prev,
                                                            (float*)act_t, c_t, (float*)y_t, B, H);
    else
      lstm_cell_fwd_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)gx_t, gh, (const __nv_bfloat16*)b_hh,
                                                                    c_prev, (__nv_bfloat16*)act_t, c_t, (__nv_bfloat16*)y_t, B, H);
    PD_LAUNCH_CHECK("lstm_cell_fwd_kernel");
  }
  return PD_OK;
}

// pd_lstm_fwd / pd_lstm_bwd on the batch rows b0 .. b0 + B - 1 of tensors that hold Bt rows per time step, whole
// sequence in one cooperative kernel: the halves of a batch, launched on two streams, run side by side on the GPU
// (the recurrence is a chain of latencies, and each half hides the other's).  bf16 only.  Returns 1 - nothing
// enqueued - where the cooperative kernels do not apply (the caller then uses pd_lstm_fwd / pd_lstm_bwd on the whole
// batch).  counter_ws: 4 bytes of device scratch per call in flight; dh_ws, dc_ws: [B, H] fp32 per call in flight.
PD_EXPORT int pd_lstm_fwd_rows(int dtype, const void* gx, const void* w_hh, const void* b_hh, int T, int Bt, int b0,
                               int B, int H, void* y, void* act, float* c_all, void* counter_ws, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(gx && w_hh && y && act && c_all && counter_ws && T > 0 && B > 0 && H > 0, "pd_lstm_fwd_rows: bad arguments");
  if (dtype != PD_BF16) return 1;
  static const bool enabled = [] { const char* e = getenv("PD_LSTM_PERSISTENT"); return !(e && e[0] == '0'); }();
  if (!enabled) return 1;
  return pd_lstm_fwd_persistent_rows(gx, w_hh, b_hh, T, Bt, b0, B, H, y, act, c_all, (unsigned int*)counter_ws,
                                     (cudaStream_t)stream);
}

PD_EXPORT int pd_lstm_bwd_rows(int dtype, const void* dy, const void* w_hh, const void* act, const float* c_all, int T,
                               int Bt, int b0, int B, int H, void* dgates, float* dh_ws, float* dc_ws, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(dy && w_hh && act && c_all && dgates && dh_ws && dc_ws && T > 0 && B > 0 && H > 0, "pd_lstm_bwd_rows: bad arguments");
  if (dtype != PD_BF16) return 1;
  static const bool enabled = [] { const char* e = getenv("PD_LSTM_PERSISTENT"); return !(e && e[0] == '0'); }();
  if (!enabled) return 1;
  return pd_lstm_bwd_persistent_rows(dy, w_hh, act, c_all, T, Bt, b0, B, H, dgates, dh_ws, dc_ws, (cudaStream_t)stream);
}

// Backward recurrence.  dy: [T,B,H]; act, c_all: saved by pd_lstm_fwd; dgates: [T,B,4H] (out) gradients
// of the gate pre-activations, from which the caller forms dx, dW_ih, dW_hh and the bias gradients with
// three contractions and a column sum.  dh_ws, dc_ws: [B,H] fp32 scratch.
PD_EXPORT int pd_lstm_bwd(int dtype, const void* dy, const void* w_hh, const void* act, const float* c_all,
                          int T, int B, int H, void* dgates, float* dh_ws, float* dc_ws, void* stream) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(dy && w_hh && act && c_all && dgates && dh_ws && dc_ws && T > 0 && B > 0 && H > 0, "pd_lstm_bwd: bad arguments");
  PD_REQUIRE(dtype == PD_F32 || dtype == PD_BF16, "pd_lstm_bwd: bad dtype");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PD_BF16) {
    static const bool enabled = [] { const char* e = getenv("PD_LSTM_PERSISTENT"); return !(e && e[0] == '0'); }();
    if (enabled) {
      const int prc = pd_lstm_bwd_persistent(dy, w_hh, act, c_all, T, B, H, dgates, dh_ws, dc_ws, s);
      if (prc != 1) return prc;
    }
  }
  const int es = pd_elem_size(dtype);
  const int64_t BH = (int64_t)B * H;
  const int grid = cell_grid(B, H);
  for (int t = T - 1; t >= 0; --t) {
    const char* dy_t = (const char*)dy + (int64_t)t * BH * es;
    const char* act_t = (const char*)act + (int64_t)t * 4 * BH * es;
    char* dg_t = (char*)dgates + (int64_t)t * 4 * BH * es;
    const float* c_t = c_all + (int64_t)t * BH;
    const float* c_prev = t > 0 ? c_all + (int64_t)(t - 1) * BH : nullptr;
    const int first = t == T - 1;
    if (dtype == PD_F32)
      lstm_cell_bwd_kernel<float><<<grid, kThreads, 0, s>>>((const float*)dy_t, dh_ws, dc_ws, (const float*)act_t, c_t,
                                                            c_prev, (float*)dg_t, B, H, first);
    else
      lstm_cell_bwd_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>((const __nv_bfloat16*)dy_t, dh_ws, dc_ws,
                                                                    (const __nv_bfloat16*)act_t, c_t, c_prev,
                                                                    (__nv_bfloat16*)dg_t, B, H, first);
    PD_LAUNCH_CHECK("lstm_cell_bwd_kernel");
    if (t > 0) {
      // dh_{t-1} (+)= dgates_t . W_hh   ([B,4H] x [4H,H]); dh_ws was cleared by the cell kernel
      PdGemm g; init_gemm(g);
      g.dtype = dtype;
      g.a = dgates; g.a_rows = (int64_t)T * B; g.a_cols = 4 * H; g.lda = 4 * H; g.a_major = 0;
      g.a_row0 = t * B;
      g.b = w_hh; g.b_rows = 4 * H; g.b_cols = H; g.ldb = H; g.b_major = 1;
      g.M = B; g.N = H; g.K = 4 * H;
      g.out = dh_ws; g.out_dtype = PD_F32; g.ldo = H;
      g.atomic = 1;
      g.split_k = dtype == PD_BF16 ? 8 : 4;
      rc = launch(g, s);
      if (rc != PD_OK) return rc;
    }
  }
  return PD_OK;
}
