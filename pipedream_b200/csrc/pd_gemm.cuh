// Internal description of one contraction launch, shared by the tcgen05 (bf16)
// and the SIMT (fp32) back ends.  The C-ABI entry points in pd_gemm_api.cu fill
// it in for Linear / 3x3-convolution forward, data-gradient and weight-gradient.
//
//   D[z][m, n] (+)= sum_{t < num_taps} sum_{k < K} A(m, t, k) * B(n, t, k)
//
// Operand A is a 2-D row-major global matrix (a_rows x a_cols, leading dim lda).
//   K-major  (a_major = 0): A(m,t,k) = a[a_row0 + m + a_tap_row[t] + z*0][a_col0 + a_tap_col[t] + k]
//   MN-major (a_major = 1): A(m,t,k) = a[a_row0 + k + a_tap_row[t]][a_col0 + a_tap_col[t] + m]
// and likewise for B with n.  Rows outside [0, rows) read as zero (this is what
// gives the convolution its zero padding at the two ends of the buffer).
// z enumerates independent outputs (the 9 taps of a weight gradient): for output
// z the B rows are additionally shifted by z_b_row[z] and the output pointer by
// z * z_out_col elements.  split_k > 1 slices the K range over extra CTAs that
// accumulate with fp32 atomics.
#pragma once
#include "pd_common.cuh"

#define PD_MAX_TAPS 9

struct PdGemm {
  int dtype;  // PD_BF16 -> tcgen05, PD_F32 -> SIMT
  const void* a; int64_t a_rows, a_cols, lda; int a_major;
  const void* b; int64_t b_rows, b_cols, ldb; int b_major;
  int M, N, K;
  int num_taps;
  int a_row0, a_col0, b_row0, b_col0;
  int a_tap_row[PD_MAX_TAPS], a_tap_col[PD_MAX_TAPS];
  int b_tap_row[PD_MAX_TAPS], b_tap_col[PD_MAX_TAPS];
  int num_z; int z_b_row[PD_MAX_TAPS]; int64_t z_out_col;
  int z_group;                // tcgen05: up to this many z outputs share one CTA (and its A tiles)
  int split_k;
  int share_tap_rows;         // tcgen05: taps 3r..3r+2 read rows that differ by 0/1/2 - let them share one A box
  // epilogue
  void* out; int out_dtype; int64_t ldo;
  int atomic;                 // fp32 atomicAdd into out (out_dtype must be PD_F32)
  const void* bias; int bias_dtype;   // per-column bias (may be null)
  int relu;                   // max(x, 0) after the bias
  int pad_hp, pad_wp;         // > 0: rows are padded-NHWC pixels, border rows are written as 0
  const void* relu_aux; int64_t ld_aux;  // != null: out = aux[m,n] > 0 ? acc : 0 (aux in out dtype)
};

int pd_gemm_launch_tcgen05(const PdGemm& g, cudaStream_t stream);
// True when the tcgen05 back end runs this problem on CTA pairs (256 x 256 tiles) rather than single CTAs.
bool pd_gemm_use_pair(int M, int N, int num_z, int z_group, int split_k);
// 128-byte-swizzle bf16 tensor map of a row-major [rows, cols] matrix (leading dim ld elements), cached per host
// thread; box = box_cols x box_rows elements (box_cols * 2 bytes <= 128).
int pd_gemm_error_word(int** out);
// Whole-sequence LSTM forward as one cooperative kernel; returns 1 when it does not apply (pd_lstm_persist.cu).
int pd_lstm_fwd_persistent(const void* gx, const void* w_hh, const void* b_hh, int T, int B, int H, void* y, void* act,
                           float* c_all, unsigned int* counter, cudaStream_t s);
int pd_lstm_bwd_persistent(const void* dy, const void* w_hh, const void* act, const float* c_all, int T, int B, int H,
                           void* dgates, float* dh_ws, float* dc_ws, cudaStream_t s);
// The same on batch rows b0 .. b0 + B - 1 of tensors holding Bt rows per time step (two halves of a batch side by side).
int pd_lstm_fwd_persistent_rows(const void* gx, const void* w_hh, const void* b_hh, int T, int Bt, int b0, int B, int H,
                                void* y, void* act, float* c_all, unsigned int* counter, cudaStream_t s);
int pd_lstm_bwd_persistent_rows(const void* dy, const void* w_hh, const void* act, const float* c_all, int T, int Bt,
                                int b0, int B, int H, void* dgates, float* dh_ws, float* dc_ws, cudaStream_t s);
struct CUtensorMap_st;
int pd_make_map_2d(CUtensorMap_st* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols,
                   int box_rows);
int pd_gemm_launch_simt(const PdGemm& g, cudaStream_t stream);
