/*
 * pipedream_b200 - C ABI of libpipedream_b200.so (CUDA, sm_100a only).
 *
 * The reference (msr-fiddle/pipedream, `pipedream` branch) reaches its GPU work through
 * PyTorch operators from Python; the only native code it ships is the pack_utils
 * extension.  This header declares what a drop-in for the training-step hot path binds
 * instead.  Each entry point names the reference call site it replaces (file:line inside
 * the reference repository).
 *
 * Conventions
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless stated
 *   - the caller owns all memory; no entry point allocates or frees device memory
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*); no hidden syncs
 *     except where stated
 *   - return value: 0 = ok, <0 = error (-1 invalid argument / unsupported shape,
 *     -2 CUDA error, -3 device is not sm_100, -4 bounded device wait ran out,
 *     -5 wrong state); pd_last_error() gives the thread-local message
 *   - dtype codes: 0 = fp32, 1 = bf16 (2 = uint8 where stated)
 *   - "padded NHWC": a logical [N,C,H,W] activation stored as [N, H+2, W+2, C] with a
 *     zero one-pixel border, C innermost; P = N*(H+2)*(W+2) pixel rows
 */
#ifndef PIPEDREAM_B200_H_
#define PIPEDREAM_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- library ------------------------------------------------------------------------- */
const char* pd_last_error(void);
int pd_abi_version(void);
int pd_device_ok(void);   /* 0 when the current device is sm_100 */
int pd_sm_count(void);

/* ---- optimizer over the weight-version ring -------------------------------------------
 * Replaces runtime/optimizer.py:122-164 (`step`: base optimizer step + push of a cloned
 * state_dict), runtime/optimizer.py:87-116 (`set_params` copies) and the per-tensor
 * torch.optim.SGD / Adam loops behind runtime/sgd.py:12-24 and runtime/adam.py:12-22.
 * arena: num_slots x slot_stride elements of w_dtype; the kernel reads slot read_slot
 * (or `master`, fp32, required when w_dtype is bf16) and writes slot write_slot, `master`
 * and the state in place.  grad is fp32 and is multiplied by grad_scale first.            */
int pd_opt_sgd_multi_tensor(void* arena, int64_t slot_stride, int read_slot, int write_slot,
                            int w_dtype, float* master, const float* grad, float* momentum_buf,
                            int64_t n, float lr, float momentum, float dampening,
                            float weight_decay, int nesterov, int first_step, float grad_scale,
                            void* stream);
int pd_opt_adam_multi_tensor(void* arena, int64_t slot_stride, int read_slot, int write_slot,
                             int w_dtype, float* master, const float* grad, float* exp_avg,
                             float* exp_avg_sq, int64_t n, float lr, float beta1, float beta2,
                             float eps, float weight_decay, int64_t step, float grad_scale,
                             void* stream);
/* x *= s; replaces `p.grad.div_(update_interval)` (runtime/optimizer.py:147-149) and the
 * gradient averaging DistributedDataParallel does for a replicated stage
 * (runtime/runtime.py:258-262).                                                            */
int pd_scale(void* x, int64_t n, int dtype, float s, void* stream);
/* dst = (dst_dtype) src; replaces apex master<->model copies (runtime/optimizer.py:137-155). */
int pd_convert(void* dst, int dst_dtype, const void* src, int src_dtype, int64_t n, void* stream);

/* ---- layout ----------------------------------------------------------------------------
 * The stage modules keep logical NCHW tensors (runtime/image_classification/models/vgg16/
 * gpus=8/stage0.py:47-71); these move data into and out of padded NHWC.                    */
int pd_pack_pnhwc(const void* src, int src_dtype, int64_t sN, int64_t sC, int64_t sH, int64_t sW,
                  int N, int C, int H, int W, void* dst, int dst_dtype, void* stream);
int pd_unpack_pnhwc(const void* src, int src_dtype, int N, int C, int H, int W, void* dst,
                    int dst_dtype, void* stream);
/* 3x3 patch matrix [P, Kpad] (k = (r*3+s)*C + c) of a small-C input: first VGG convolution. */
int pd_im2col3x3(const void* src, int src_dtype, int64_t sN, int64_t sC, int64_t sH, int64_t sW,
                 int N, int C, int H, int W, int Kpad, void* dst, int dst_dtype, void* stream);

/* ---- pointwise -------------------------------------------------------------------------
 * torch.nn.ReLU / MaxPool2d(2,2) / Dropout of the stage files (vgg16/gpus=8/stage0.py:11-31,
 * stage1.py:10-25), forward and backward.                                                  */
int pd_relu_fwd(const void* x, void* y, int64_t n, int dtype, void* stream);
int pd_relu_bwd(const void* dy, const void* y, void* dx, int64_t n, int dtype, void* stream);
int64_t pd_colsum_workspace_bytes(int C);
/* dx = dy * (y > 0) (y, dx may be NULL) and colsum[C] (+)= column sums: ReLU backward fused
 * with the bias gradient of the Conv2d / Linear in front of it.  workspace: scratch of at
 * least pd_colsum_workspace_bytes(C) bytes.                                                */
int pd_relu_bwd_colsum(const void* dy, const void* y, void* dx, int64_t rows, int C, int dtype,
                       float* colsum, int accumulate, void* workspace, int64_t workspace_bytes,
                       void* stream);
/* out_mode / dy_mode: 0 = padded NHWC, 1 = contiguous NCHW.                                */
int pd_maxpool2_fwd(const void* x_pad, int N, int C, int H, int W, void* y, int out_mode,
                    int dtype, void* stream);
int pd_maxpool2_bwd(const void* x_pad, const void* dy, int N, int C, int H, int W, void* dx_pad,
                    int dy_mode, int relu_mask, int dtype, void* stream);
/* The same backward (dy in padded NHWC) that also reduces the bias gradient of the convolution in
 * front of the pool: block b leaves the column sums of the gradient it routed in partial[b][C]
 * (*partial_rows rows; partial holds at least pd_colsum_workspace_bytes(C) bytes), and
 * pd_colsum_finish adds the rows into out[C].  Needs bf16, even H and W, C % 8 == 0 with
 * 256 % (C / 8) == 0 and 16-byte aligned pointers (PD_ERR_INVALID otherwise).               */
int pd_maxpool2_bwd_colsum(const void* x_pad, const void* dy_pad, int N, int C, int H, int W,
                           void* dx_pad, int relu_mask, int dtype, float* partial,
                           int64_t partial_bytes, int* partial_rows, void* stream);
int pd_colsum_finish(const float* partial, int rows, int C, float* out, int accumulate, void* stream);
int pd_dropout_fwd(const void* x, void* y, uint8_t* mask, int64_t n, float p, uint64_t seed,
                   uint64_t offset, int dtype, void* stream);
int pd_dropout_bwd(const void* dy, const uint8_t* mask, void* dx, int64_t n, float p, int dtype,
                   void* stream);
/* y = a + b: residual adds of the ResNet-50 / GNMT stage files.                             */
int pd_add(const void* a, const void* b, void* y, int64_t n, int dtype, void* stream);

/* torch.nn.BatchNorm2d of the ResNet-50 stages (runtime/image_classification/models/resnet50/gpus=4/
 * stage1.py:12-55; cuDNN batch norm in the reference), on padded NHWC.  Training forward computes the
 * batch statistics (mean, invstd: fp32 [C], saved), updates running_mean / running_var like torch
 * (momentum, unbiased variance), applies gamma/beta, then optionally adds res_pad (the shortcut of a
 * bottleneck block, stage1.py forward: `out = out + identity`) and applies the ReLU that follows.
 * Backward takes the saved statistics; y_pad != NULL means the forward applied a ReLU; dres_pad (may be
 * NULL) receives the masked dy, the gradient of the residual input.  workspace: fp32 scratch of
 * pd_bn_workspace_bytes(C) bytes; sums_ws: fp32 [2*C].  C <= 2048.                                 */
int64_t pd_bn_workspace_bytes(int C);
int pd_bn_fwd(int dtype, const void* x_pad, const void* res_pad, int N, int H, int W, int C, const void* gamma,
              const void* beta, float eps, float momentum, int relu, float* mean, float* invstd, float* running_mean,
              float* running_var, void* y_pad, void* workspace, int64_t workspace_bytes, void* stream);
int pd_bn_apply(int dtype, const void* x_pad, const void* res_pad, int N, int H, int W, int C, const void* gamma,
                const void* beta, const float* mean, const float* invstd, int relu, void* y_pad, void* stream);
int pd_bn_bwd(int dtype, const void* x_pad, const void* dy_pad, const void* y_pad, int N, int H, int W, int C,
              const void* gamma, const float* mean, const float* invstd, float* dgamma, float* dbeta,
              int accumulate, void* dx_pad, void* dres_pad, float* sums_ws, void* workspace,
              int64_t workspace_bytes, void* stream);
/* Convolution variants other than 3x3/stride 1 (resnet50/gpus=4/stage0.py:10: 7x7 stride 2; 1x1 and 3x3
 * stride 2) run as a patch matrix through pd_gemm_*: pd_im2col builds [N*Ho*Wo, Kpad] (k = (r*kw+s)*C + c)
 * from an any-stride NCHW source, pd_col2im_pnhwc gathers the patch-matrix gradient back into padded NHWC. */
int pd_im2col(const void* src, int src_dtype, int64_t sN, int64_t sC, int64_t sH, int64_t sW, int N, int C,
              int H, int W, int kh, int kw, int stride, int pad, int Ho, int Wo, int Kpad, void* dst,
              int dst_dtype, void* stream);
int pd_col2im_pnhwc(const void* dcol, int N, int C, int H, int W, int kh, int kw, int stride, int pad, int Ho,
                    int Wo, int Kpad, void* dx_pad, int dtype, void* stream);
/* MaxPool2d(3, stride 2, padding 1) and the global AvgPool2d(7) of resnet50 (stage0.py:13, stage2.py),
 * padded NHWC in; the average pool writes / reads a contiguous [N, C] matrix.                       */
int pd_maxpool3s2_fwd(const void* x_pad, int N, int C, int H, int W, void* y_pad, unsigned char* argmax, int dtype,
                      void* stream);   /* argmax: [N,Ho,Wo,C] bytes (position r*3+s of the window maximum) or NULL */
int pd_maxpool3s2_bwd(const unsigned char* argmax, const void* dy_pad, int N, int C, int H, int W, void* dx_pad,
                      int dtype, void* stream);
int pd_avgpool_fwd(const void* x_pad, int N, int C, int H, int W, void* y, int dtype, void* stream);
int pd_avgpool_bwd(const void* dy, int N, int C, int H, int W, void* dx_pad, int dtype, void* stream);

/* ---- criteria --------------------------------------------------------------------------
 * torch.nn.CrossEntropyLoss (runtime/image_classification/main_with_runtime.py:126) and
 * LabelSmoothing (runtime/translation/seq2seq/train/smoothing.py:23-34).  smoothing = 0 and
 * padding_idx < 0 give plain cross-entropy.  loss = scale * sum(row_loss).  row_loss[rows]
 * and lse[rows] are caller-provided scratch / saved statistics.                             */
int pd_softmax_ce_fwd(const void* logits, int dtype, const int64_t* target, int64_t rows, int C,
                      float smoothing, int64_t padding_idx, float scale, float* row_loss,
                      float* lse, float* loss, void* stream);
int pd_softmax_ce_bwd(const void* logits, int dtype, const int64_t* target, const float* lse,
                      int64_t rows, int C, float smoothing, int64_t padding_idx,
                      const float* upstream, float gscale, void* dlogits, void* stream);

/* No counterpart in the reference: the forward criterion for callers that must not allocate.
 * Identical result to pd_softmax_ce_fwd, but the per-row scratch is a fixed 65536-row array
 * inside the library (256 KiB held by every GPU that loads it) and the call performs no device
 * allocation.  Meant for hosts with a fixed device-memory plan (all HBM handed out up front) or
 * a no-allocation rule after start-up.  rows > pd_softmax_ce_static_max_rows() is an error (-1).
 * The first call on a device looks up the array's address: make it before any stream capture.
 * Calls share the array; calls that overlap on the GPU race.                                  */
int pd_softmax_ce_fwd_static(const void* logits, int dtype, const int64_t* target, int64_t rows,
                             int C, float smoothing, int64_t padding_idx, float scale, float* lse,
                             float* loss, void* stream);
int64_t pd_softmax_ce_static_max_rows(void);

/* ---- sequence utilities ----------------------------------------------------------------
 * pd_revert_varlen replaces revert_varlen_tensor (runtime/translation/seq2seq/csrc/
 * pack_utils_kernel.cu:24-63); pd_length_mask replaces set_mask_cpp (csrc/pack_utils.cpp:
 * 13-31).  `lengths` is an int64 DEVICE vector here (the reference takes a CPU tensor and
 * rebuilds and uploads an offset table on every call).  mask_dtype 2 = uint8.               */
int pd_revert_varlen(const void* in, void* out, const int64_t* lengths, int T, int B,
                     int64_t feature_bytes, void* stream);
int pd_length_mask(const int64_t* lengths, int T, int B, void* mask, int mask_dtype, void* stream);
/* y[r,:] = x[r,:] * mask[r] (mask in the tensor's dtype): `model0(input)[0] * mask` of
 * runtime/translation/seq2seq/models/encoder.py:51,55.                                          */
int pd_mul_rows(const void* x, const void* mask, void* y, int64_t rows, int F, int dtype, void* stream);
/* torch.nn.Embedding(padding_idx=0) of runtime/translation/models/gnmt_large/gpus=4/stage0.py:10 */
int pd_embedding_fwd(const int64_t* ids, const void* table, int64_t n, int D, int64_t vocab,
                     void* out, int dtype, void* stream);
int pd_embedding_bwd(const int64_t* ids, const void* dy, int64_t n, int D, int64_t vocab,
                     int64_t padding_idx, float* dtable, int dtype, void* stream);

/* ---- contractions ----------------------------------------------------------------------
 * bf16 problems run on tcgen05 tensor cores (TMA-fed, fp32 accumulation in tensor memory),
 * fp32 problems on CUDA cores.  Leading dimensions are in elements; for bf16 they must be
 * multiples of 8 and base pointers 16-byte aligned.
 *
 * pd_gemm_nt : out[M,N] = a[M,K] . b[N,K]^T (+bias[N]) (ReLU)  - torch.nn.Linear forward
 *              (vgg16/gpus=16/stage1.py:10-16).  pad_hp/pad_wp > 0: rows are padded-NHWC
 *              pixels and border rows are written as zero.
 * pd_gemm_nn : out[M,N] = a[M,K] . b[K,N], optionally masked by (relu_aux[M,N] > 0)
 *              - Linear data gradient.
 * pd_gemm_tn : out[M,N] (fp32) (+)= a[K,M]^T . b[K,N]           - Linear weight gradient.
 *              split_k = 0 picks a split; partial sums are combined with fp32 atomics.      */
int pd_gemm_nt(int dtype, const void* a, int64_t lda, const void* b, int64_t ldb, void* out,
               int out_dtype, int64_t ldo, int M, int N, int K, const void* bias, int bias_dtype,
               int relu, int pad_hp, int pad_wp, void* stream);
/* pd_gemm_nt for a short, wide problem (a Linear layer at a batch of 64: a handful of output tiles,
 * hundreds of MB of weights): K is cut into slices that add into `workspace`
 * (pd_gemm_nt_splitk_workspace_bytes(M, N) bytes of device memory, cleared by the call) with fp32
 * atomics, then bias / ReLU / conversion into `out`.  bf16 operands only.                       */
int64_t pd_gemm_nt_splitk_workspace_bytes(int M, int N);
int pd_gemm_nt_splitk(int dtype, const void* a, int64_t lda, const void* b, int64_t ldb, void* out,
                      int out_dtype, int64_t ldo, int M, int N, int K, const void* bias,
                      int bias_dtype, int relu, void* workspace, int64_t workspace_bytes,
                      void* stream);
int pd_gemm_nn(int dtype, const void* a, int64_t lda, const void* b, int64_t ldb, void* out,
               int out_dtype, int64_t ldo, int M, int N, int K, const void* relu_aux,
               int64_t ld_aux, void* stream);
int pd_gemm_tn(int dtype, const void* a, int64_t lda, const void* b, int64_t ldb, float* out,
               int64_t ldo, int M, int N, int K, int accumulate, int split_k, void* stream);
/* torch.nn.Conv2d(kernel 3x3, stride 1, padding 1) forward / input gradient / weight gradient
 * (vgg16/gpus=8/stage0.py:10-31, stage1.py:12-16) as implicit GEMMs over padded NHWC.
 * w: [Cout][3][3][Cin] (channels-last order of the [Cout,Cin,3,3] parameter), leading dim ldw.
 * dgrad: relu_aux != NULL additionally multiplies dx by (relu_aux > 0), relu_aux = the
 * padded-NHWC input of the layer.  wgrad: dw fp32 [Cout][9*Cin], leading dim lddw.          */
int pd_conv2d_fwd(int dtype, const void* x_pad, int N, int H, int W, int Cin, const void* w,
                  int64_t ldw, int Cout, const void* bias, int bias_dtype, int relu, void* y_pad,
                  void* stream);
int pd_conv2d_dgrad(int dtype, const void* dy_pad, int N, int H, int W, int Cout, const void* w,
                    int64_t ldw, int Cin, const void* relu_aux, void* dx_pad, void* stream);
int pd_conv2d_wgrad(int dtype, const void* x_pad, const void* dy_pad, int N, int H, int W, int Cin,
                    int Cout, float* dw, int64_t lddw, int accumulate, int split_k, void* stream);
/* torch.nn.LayerNorm over the last dimension and torch.nn.GELU, for transformer stage modules (the 2BW
 * configuration; the reference itself ships no such stage files, its runtime would reach ATen's kernels through
 * torch.nn).  x, y, dy, dx: [rows, C] (C <= 1024); gamma, beta in `dtype`; mean, rstd: fp32 [rows] saved by the
 * forward; dgamma, dbeta: fp32 [C], stored or accumulated; workspace: pd_layernorm_workspace_bytes(rows, C) bytes.
 * GELU: tanh_form != 0 selects the tanh approximation, else the erf form.                                       */
int64_t pd_layernorm_workspace_bytes(int64_t rows, int C);
int pd_layernorm_fwd(int dtype, const void* x, int64_t rows, int C, const void* gamma, const void* beta, float eps,
                     void* y, float* mean, float* rstd, void* stream);
int pd_layernorm_bwd(int dtype, const void* x, const void* dy, const void* gamma, const float* mean,
                     const float* rstd, int64_t rows, int C, void* dx, float* dgamma, float* dbeta, int accumulate,
                     void* workspace, int64_t workspace_bytes, void* stream);
int pd_gelu_fwd(int dtype, const void* x, void* y, int64_t n, int tanh_form, void* stream);
int pd_gelu_bwd(int dtype, const void* x, const void* dy, void* dx, int64_t n, int tanh_form, void* stream);
/* Causal self-attention of a transformer block, softmax(Q K^T scale) V per head (the PipeDream-2BW GPT stages; the
 * reference tree holds no transformer stage files).  qkv [B, T, 3, H, d]: the fused projection's output, read in
 * place; out [B, T, H*d]; probs [B*H, T, T]: the attention weights, kept for the backward pass.  Backward: dqkv
 * [B, T, 3, H, d] from dout [B, T, H*d]; dscores [B*H, T, T] is scratch.  bf16, d == 64, T a multiple of 128 up to
 * 2048 (PD_ERR_INVALID otherwise).                                                                            */
int pd_sdpa_causal_fwd(int dtype, const void* qkv, int B, int T, int H, int d, float scale, void* out,
                       void* probs, void* stream);
int pd_sdpa_causal_bwd(int dtype, const void* qkv, const void* probs, const void* dout, int B, int T, int H,
                       int d, float scale, void* dqkv, void* dscores, void* stream);
/* torch.nn.LSTM(I, H), one layer, one direction, [T,B,*] sequences (runtime/translation/models/
 * gnmt_large/gpus=4/stage0.py:11-19; the reference reaches cuDNN's RNN through it): the time loop.
 * The caller computes the input projections gx = x . W_ih^T + b_ih for all steps with pd_gemm_nt;
 * pd_lstm_fwd then runs, per step, h_{t-1} . W_hh^T on the tensor cores and a fused cell kernel
 * (gate order i,f,g,o; cell state kept in fp32; zero initial state), saving gate activations `act`
 * [T,B,4H] and cell states `c_all` [T,B,H] (fp32).  pd_lstm_bwd walks back through time and
 * produces the gate pre-activation gradients `dgates` [T,B,4H]; dx, dW_ih, dW_hh and the bias
 * gradients are then pd_gemm_nn / pd_gemm_tn / pd_relu_bwd_colsum calls over dgates.
 * gh_ws [B,4H], dh_ws and dc_ws [B,H]: fp32 scratch provided by the caller.
 * In bf16 with B <= 128 the recurrences run as ONE cooperative kernel per call where the sizes allow
 * (forward: H a multiple of 64, H/8 <= number of SMs; backward: H a power of two in 128..1024): weights
 * stay in shared memory for the whole sequence, the cell update is fused in, steps are separated by a
 * grid-wide counter; results and saved tensors are the same.  PD_LSTM_PERSISTENT=0 in the environment
 * selects the per-step launches everywhere.                                                            */
int pd_lstm_fwd(int dtype, const void* gx, const void* w_hh, const void* b_hh, int T, int B, int H,
                void* y, void* act, float* c_all, float* gh_ws, void* stream);
int pd_lstm_bwd(int dtype, const void* dy, const void* w_hh, const void* act, const float* c_all,
                int T, int B, int H, void* dgates, float* dh_ws, float* dc_ws, void* stream);

/* The two recurrences on the batch rows b0 .. b0 + B - 1 of tensors that hold Bt rows per time step (bf16, whole
 * sequence in one cooperative kernel): the halves of a batch, launched on two streams, run side by side.  Return 1,
 * with nothing enqueued, where the cooperative kernels do not apply - call pd_lstm_fwd / pd_lstm_bwd on the whole
 * batch then.  counter_ws: 4 bytes of device scratch; dh_ws, dc_ws: [B, H] fp32, per call in flight.          */
int pd_lstm_fwd_rows(int dtype, const void* gx, const void* w_hh, const void* b_hh, int T, int Bt, int b0, int B,
                     int H, void* y, void* act, float* c_all, void* counter_ws, void* stream);
int pd_lstm_bwd_rows(int dtype, const void* dy, const void* w_hh, const void* act, const float* c_all, int T, int Bt,
                     int b0, int B, int H, void* dgates, float* dh_ws, float* dc_ws, void* stream);

/* Normalised additive attention (runtime/translation/seq2seq/models/attention.py:84-170:
 * `calc_score`, mask, softmax, `bmm`) fused so that tanh(q + k + b) is never stored.  pq [b,tq,n] and
 * pk [b,tk,n] are the projected queries / keys (pd_gemm_nt); v [n] fp32 is linear_att / |linear_att| *
 * normalize_scalar; nb [n] is normalize_bias; ctx_len [b] int64 masks keys j >= ctx_len[b] (score
 * -65504 as in the reference) or NULL.  keys / context / dkeys are addressed as base + batch*sb +
 * time*st + channel (elements), so sequence-first tensors are used in place.  tk <= 128.
 * Backward: dv, dnb fp32 [n] are accumulated into (clear them first); ds_ws [b,tq,tk] fp32 scratch.  */
int pd_attn_bahdanau_fwd(int dtype, const void* pq, const void* pk, const void* keys, int64_t k_sb,
                         int64_t k_st, const float* v, const void* nb, const int64_t* ctx_len, int b,
                         int tq, int tk, int n, int nk, void* probs, void* context, int64_t c_sb,
                         int64_t c_st, void* stream);
int pd_attn_bahdanau_bwd(int dtype, const void* pq, const void* pk, const void* keys, int64_t k_sb,
                         int64_t k_st, const float* v, const void* nb, const void* probs,
                         const void* dcontext, int64_t c_sb, int64_t c_st, int b, int tq, int tk, int n,
                         int nk, void* dpq, void* dpk, void* dkeys, int64_t dk_sb, int64_t dk_st,
                         float* dv, float* dnb, float* ds_ws, void* stream);

/* Reads and clears the error word the tcgen05 kernels set when a bounded wait runs out
 * (0 = none).  `code` is a HOST pointer; synchronises the device.                            */
int pd_gemm_poll_error(int* code);
/* Tiling switch of the bf16 contraction back end.  mode 1 (default): problems whose output is at least
 * 256 x 256 with N a multiple of 256 (the 256- and 512-channel convolutions of vgg16/gpus=8/stage0.py:16-31
 * in all three passes) run on pairs of CTAs - a cluster of two SMs sharing one 256 x 256 tile through
 * tcgen05.mma.cta_group::2 - and the 64- and 128-channel convolutions run two 128-row groups per tile, each with
 * its own MMA-issuing warp (the 128-channel ones on CTA pairs as well); mode 0: every problem runs on single CTAs
 * with one group (128-row tiles); mode 3: pairs, but one group.  All tilings add the same products in the same
 * order.  Process-wide; meant for checking one tiling against the other.                                      */
int pd_gemm_set_pair_mode(int mode);
/* Diagnostic for the bf16 contraction kernel (no counterpart in the reference): with `device_buffer` pointing at
 * 4 x (SM count) int64 in device memory, the MMA-issuing warp of every CTA adds, per launch, {cycles waiting for
 * operand tiles to land in shared memory, cycles waiting for the epilogue to free an accumulator, total cycles,
 * tiles} to its four slots.  NULL (the default) switches the counters off.  Process-wide.                    */
int pd_gemm_set_stall_counters(void* device_buffer);

/* ---- peer channels --------------------------------------------------------------------
 * One-directional FIFO between two pipeline-adjacent GPUs; replaces the helper threads and the
 * GPU -> CPU -> TCP -> CPU -> GPU path of runtime/communication.py:610-712 (`recv_helper_thread`,
 * `send_helper_thread`, `_recv`, `_send`) and the shape message of :664-669.  The ring of
 * `num_slots` slots lives in the consumer's HBM and is mapped into the producer process with
 * CUDA IPC; a push is wait-for-free-slot, NVLink copy, publish, all enqueued on `stream`.
 * create/open/close are set-up calls (they allocate and synchronise); push and wait are not.
 * timeout_ms bounds every device-side wait; when it runs out the channel's status becomes -4
 * and the kernels return, so a dead peer cannot hang the GPU.  A receive whose byte count differs
 * from the message's sets status -1.  A channel with a non-zero status is dead: queued waits return
 * at once, no payload is copied into a slot that was not freed, nothing is published or released,
 * and a receive zero-fills its destination.  pd_chan_status synchronises `stream` and returns the
 * status; pd_chan_poll returns it from a pinned host mirror without touching any stream.
 * blob128: 128 bytes of HOST memory carried to the producer by any host transport.
 * pd_chan_open_local makes a producer end over the same memory inside one process (tests).
 * pd_chan_peek_header blocks the host until the next message is there; out8 (HOST) receives
 * {seq, nbytes, ndim, d0..d4} - for tensors whose shape changes per minibatch.               */
int pd_chan_create(int64_t slot_bytes, int num_slots, int timeout_ms, void** chan);
int pd_chan_export_handle(void* chan, void* blob128);
int pd_chan_open(const void* blob128, int timeout_ms, void** chan);
int pd_chan_open_local(void* consumer_chan, int timeout_ms, void** chan);
int pd_chan_push(void* chan, const void* src, int64_t bytes, int ndim, const int64_t* dims,
                 void* stream);
int pd_chan_wait(void* chan, void* dst, int64_t bytes, void* stream);
int pd_chan_peek_header(void* chan, int64_t* out8, void* stream);
int pd_chan_status(void* chan, void* stream);
int pd_chan_poll(void* chan);
int pd_chan_close(void* chan);

#ifdef __cplusplus
}
#endif
#endif /* PIPEDREAM_B200_H_ */
