"""Tensor-level wrappers over the C-ABI kernels (no autograd here).

Every function takes CUDA tensors, passes raw device pointers and the current
CUDA stream to libpipedream_b200.so, and returns / fills torch tensors that
only serve as device-memory handles.  Nothing in this module computes with
torch operators.
"""
import ctypes
import os

import torch

from . import _lib
from ._lib import PD_BF16, PD_F32, call

_DT = {torch.float32: PD_F32, torch.bfloat16: PD_BF16}


def dt(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise _lib.PipedreamB200Error("unsupported dtype %s (fp32 and bf16 only)" % t.dtype)


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_CUR_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream of the current device as a raw handle (every entry point takes one).  The two private
    torch accessors avoid building a torch.cuda.Stream object per call; the public path is the fallback."""
    if _RAW_STREAM is not None and _CUR_DEVICE is not None:
        return ctypes.c_void_p(_RAW_STREAM(_CUR_DEVICE()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class ContractionTimeline:
    """Optional CUDA-event record of every contraction launch (benchmarks read it to get the
    achieved FLOP rate of the tensor-core kernel).  Off unless `timeline` is set."""

    def __init__(self):
        self.records = []     # (name, flops, start_event, end_event)

    def begin(self):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def end(self, name, flops, start, detail=None):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.records.append((name, flops, start, e, detail))

    def summary(self):
        """{name: (launches, total_flops, total_ms)} - call after a synchronize."""
        out = {}
        for name, flops, s, e, _ in self.records:
            n, f, t = out.get(name, (0, 0.0, 0.0))
            out[name] = (n + 1, f + flops, t + s.elapsed_time(e))
        return out

    def per_shape(self):
        """{(name, detail): (launches, total_flops, total_ms)} - call after a synchronize."""
        out = {}
        for name, flops, s, e, detail in self.records:
            k = "%s %s" % (name, detail)
            n, f, t = out.get(k, (0, 0.0, 0.0))
            out[k] = (n + 1, f + flops, t + s.elapsed_time(e))
        return out


timeline = None


def _timed(name, flops, fn, detail=None):
    if timeline is None:
        return fn()
    s = timeline.begin()
    r = fn()
    timeline.end(name, flops, s, detail)
    return r


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _lib.PipedreamB200Error("pipedream_b200 kernels need CUDA tensors (no CPU path)")


# --------------------------------------------------------------------------- #
# padded-NHWC layout helpers
# --------------------------------------------------------------------------- #
def padded_shape(N, C, H, W):
    return (N, H + 2, W + 2, C)


def nchw_view(pad, N, C, H, W):
    """Logical [N,C,H,W] view of the interior of a padded-NHWC buffer."""
    Hp, Wp = H + 2, W + 2
    return pad.as_strided((N, C, H, W), (Hp * Wp * C, 1, Wp * C, C), pad.storage_offset() + (Wp + 1) * C)


def padded_of(view):
    """If `view` is a logical-NCHW view of a padded-NHWC buffer, return that buffer, else None."""
    if view.dim() != 4:
        return None
    N, C, H, W = view.shape
    Hp, Wp = H + 2, W + 2
    if view.stride() != (Hp * Wp * C, 1, Wp * C, C):
        return None
    off = view.storage_offset() - (Wp + 1) * C
    if off < 0:
        return None
    nbytes = view.untyped_storage().nbytes() // view.element_size()
    if off + N * Hp * Wp * C > nbytes:
        return None
    return view.as_strided((N, Hp, Wp, C), (Hp * Wp * C, Wp * C, C, 1), off)


def pack_pnhwc(x, dtype=None):
    """Any-stride [N,C,H,W] tensor -> new padded-NHWC buffer (zero border)."""
    _cuda(x)
    N, C, H, W = x.shape
    dtype = dtype or x.dtype
    out = torch.empty(padded_shape(N, C, H, W), dtype=dtype, device=x.device)
    sN, sC, sH, sW = x.stride()
    call("pd_pack_pnhwc", _p(x), dt(x), sN, sC, sH, sW, N, C, H, W, _p(out), _DT[dtype], _stream())
    return out


def as_padded(x, dtype=None):
    """Padded-NHWC buffer for a logical NCHW tensor: zero-copy when it already is one."""
    pad = padded_of(x)
    if pad is not None and (dtype is None or dtype == x.dtype):
        return pad
    return pack_pnhwc(x, dtype)


def unpack_pnhwc(pad, dtype=None):
    """Padded-NHWC buffer -> contiguous NCHW tensor."""
    _cuda(pad)
    N, Hp, Wp, C = pad.shape
    H, W = Hp - 2, Wp - 2
    dtype = dtype or pad.dtype
    out = torch.empty((N, C, H, W), dtype=dtype, device=pad.device)
    call("pd_unpack_pnhwc", _p(pad), dt(pad), N, C, H, W, _p(out), _DT[dtype], _stream())
    return out


def im2col3x3(x, kpad, dtype):
    """[N,C,H,W] any-stride -> [N*(H+2)*(W+2), kpad] patch matrix over padded pixel rows."""
    _cuda(x)
    N, C, H, W = x.shape
    out = torch.empty((N * (H + 2) * (W + 2), kpad), dtype=dtype, device=x.device)
    sN, sC, sH, sW = x.stride()
    call("pd_im2col3x3", _p(x), dt(x), sN, sC, sH, sW, N, C, H, W, kpad, _p(out), _DT[dtype], _stream())
    return out


# --------------------------------------------------------------------------- #
# pointwise
# --------------------------------------------------------------------------- #
def relu_(x):
    """In-place ReLU over a dense buffer (padded buffers stay valid: relu(0) = 0)."""
    _cuda(x)
    call("pd_relu_fwd", _p(x), _p(x), x.numel(), dt(x), _stream())
    return x


def relu(x):
    y = torch.empty_like(x)
    call("pd_relu_fwd", _p(x), _p(y), x.numel(), dt(x), _stream())
    return y


def relu_bwd(dy, y, out=None):
    out = torch.empty_like(dy) if out is None else out
    call("pd_relu_bwd", _p(dy), _p(y), _p(out), dy.numel(), dt(dy), _stream())
    return out


_WS = {}


def _workspace(device, nbytes):
    key = (device.index, _stream().value)
    ws = _WS.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _WS[key] = ws
    return ws


def relu_bwd_colsum(dy, y, dx, colsum, accumulate):
    """dx = dy * (y > 0) (y, dx may be None) and colsum[C] (+)= column sums of the masked dy.

    dy is a dense [rows, C] matrix (any leading shape, C innermost)."""
    _cuda(dy, colsum)
    C = dy.shape[-1]
    rows = dy.numel() // C
    nbytes = _lib.load().pd_colsum_workspace_bytes(C)
    ws = _workspace(dy.device, nbytes)
    call("pd_relu_bwd_colsum", _p(dy), _p(y), _p(dx), rows, C, dt(dy), _p(colsum), int(accumulate), _p(ws),
         ws.numel(), _stream())


def maxpool2_fwd(x_pad, to_nchw):
    N, Hp, Wp, C = x_pad.shape
    H, W = Hp - 2, Wp - 2
    if to_nchw:
        y = torch.empty((N, C, H // 2, W // 2), dtype=x_pad.dtype, device=x_pad.device)
    else:
        y = torch.empty(padded_shape(N, C, H // 2, W // 2), dtype=x_pad.dtype, device=x_pad.device)
    call("pd_maxpool2_fwd", _p(x_pad), N, C, H, W, _p(y), 1 if to_nchw else 0, dt(x_pad), _stream())
    return y


def maxpool2_bwd(x_pad, dy, dy_is_nchw, relu_mask):
    N, Hp, Wp, C = x_pad.shape
    dx = torch.empty_like(x_pad)
    call("pd_maxpool2_bwd", _p(x_pad), _p(dy), N, C, Hp - 2, Wp - 2, _p(dx), 1 if dy_is_nchw else 0,
         int(relu_mask), dt(x_pad), _stream())
    return dx


def maxpool2_bwd_colsum_ok(x_pad):
    """Whether pd_maxpool2_bwd_colsum takes this tensor (bf16, even H and W, channel count it supports)."""
    N, Hp, Wp, C = x_pad.shape
    return (x_pad.dtype == torch.bfloat16 and Hp % 2 == 0 and Wp % 2 == 0 and C % 8 == 0 and 256 % (C // 8) == 0)


def maxpool2_bwd_colsum(x_pad, dy_pad, relu_mask):
    """Max-pool backward plus per-block column sums of dx: returns (dx_pad, (partial, rows)) for `colsum_finish`."""
    N, Hp, Wp, C = x_pad.shape
    dx = torch.empty_like(x_pad)
    nbytes = _lib.load().pd_colsum_workspace_bytes(C)
    partial = torch.empty(nbytes // 4, dtype=torch.float32, device=x_pad.device)
    rows = ctypes.c_int(0)
    call("pd_maxpool2_bwd_colsum", _p(x_pad), _p(dy_pad), N, C, Hp - 2, Wp - 2, _p(dx), int(relu_mask), dt(x_pad),
         _p(partial), nbytes, ctypes.byref(rows), _stream())
    return dx, (partial, rows.value)


def colsum_finish(partial_rows, colsum, accumulate):
    partial, rows = partial_rows
    call("pd_colsum_finish", _p(partial), rows, colsum.numel(), _p(colsum), int(accumulate), _stream())


def dropout_fwd(x, p, seed, offset):
    y = torch.empty_like(x)
    mask = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    call("pd_dropout_fwd", _p(x), _p(y), _p(mask), x.numel(), float(p), int(seed), int(offset), dt(x), _stream())
    return y, mask


def dropout_bwd(dy, mask, p):
    dx = torch.empty_like(dy)
    call("pd_dropout_bwd", _p(dy), _p(mask), _p(dx), dy.numel(), float(p), dt(dy), _stream())
    return dx


def add(a, b):
    y = torch.empty_like(a)
    call("pd_add", _p(a), _p(b), _p(y), a.numel(), dt(a), _stream())
    return y


def convert(src, dtype, out=None):
    out = torch.empty(src.shape, dtype=dtype, device=src.device) if out is None else out
    call("pd_convert", _p(out), _DT[out.dtype], _p(src), dt(src), src.numel(), _stream())
    return out


def scale_(x, s):
    call("pd_scale", _p(x), x.numel(), dt(x), float(s), _stream())
    return x


# --------------------------------------------------------------------------- #
# contractions
# --------------------------------------------------------------------------- #
def gemm_nt(a, b, bias=None, relu=False, out_dtype=None, pad_hw=None):
    """a[M,K] . b[N,K]^T (+bias) (ReLU).  pad_hw=(Hp, Wp): rows are padded pixels, border rows -> 0."""
    _cuda(a, b)
    M, K = a.shape
    N = b.shape[0]
    out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    hp, wp = pad_hw if pad_hw is not None else (0, 0)
    if (a.dtype == torch.bfloat16 and 32 <= M <= 128 and pad_hw is None and K >= 4096 and N <= 16384
            and out.dtype in (torch.bfloat16, torch.float32) and not _DETERMINISTIC):
        # a few output tiles and a long contraction (a Linear layer at a small batch): split along K over all SMs
        ws = torch.empty(M * N, dtype=torch.float32, device=a.device)
        _timed("gemm_nt", 2.0 * M * N * K, lambda: call(
            "pd_gemm_nt_splitk", dt(a), _p(a), a.stride(0), _p(b), b.stride(0), _p(out), _DT[out.dtype], out.stride(0),
            M, N, K, _p(bias), dt(bias) if bias is not None else 0, int(relu), _p(ws), ws.numel() * 4, _stream()),
            (M, N, K))
        return out
    _timed("gemm_nt", 2.0 * M * N * K, lambda: call(
        "pd_gemm_nt", dt(a), _p(a), a.stride(0), _p(b), b.stride(0), _p(out), _DT[out.dtype], out.stride(0), M, N, K,
        _p(bias), dt(bias) if bias is not None else 0, int(relu), hp, wp, _stream()), (M, N, K))
    return out


def gemm_nn(a, b, relu_aux=None):
    """a[M,K] . b[K,N], optionally masked by (relu_aux > 0)."""
    _cuda(a, b)
    M, K = a.shape
    N = b.shape[1]
    out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    _timed("gemm_nn", 2.0 * M * N * K, lambda: call(
        "pd_gemm_nn", dt(a), _p(a), a.stride(0), _p(b), b.stride(0), _p(out), _DT[out.dtype], out.stride(0), M, N, K,
        _p(relu_aux), relu_aux.stride(0) if relu_aux is not None else 0, _stream()), (M, N, K))
    return out


_DETERMINISTIC = False


def set_deterministic(flag):
    """Weight gradients are normally split along their long contraction (the pixels / tokens of the minibatch) over
    several CTAs that add their parts with fp32 atomics, in an order that changes from run to run (last-bit
    differences).  With this switch every weight gradient is computed without the split: bit-identical from run to
    run, and several times slower for the layers with few output tiles.  Returns the previous setting."""
    global _DETERMINISTIC
    prev, _DETERMINISTIC = _DETERMINISTIC, bool(flag)
    return prev


def gemm_tn(a, b, out, accumulate=False, split_k=0):
    """out[M,N] (fp32, any leading dim) (+)= a[K,M]^T . b[K,N]."""
    _cuda(a, b, out)
    if _DETERMINISTIC and split_k == 0:
        split_k = 1
    K, M = a.shape
    N = b.shape[1]
    assert out.dtype == torch.float32
    _timed("gemm_tn", 2.0 * M * N * K, lambda: call(
        "pd_gemm_tn", dt(a), _p(a), a.stride(0), _p(b), b.stride(0), _p(out), out.stride(0), M, N, K,
        int(accumulate), int(split_k), _stream()), (M, N, K))
    return out


def conv2d_fwd(x_pad, w, ldw, cout, bias, relu):
    """3x3/s1/p1 convolution on padded NHWC.  w: [Cout][r][s][Cin] storage with leading dim ldw."""
    N, Hp, Wp, Cin = x_pad.shape
    y = torch.empty((N, Hp, Wp, cout), dtype=x_pad.dtype, device=x_pad.device)
    # algorithmic FLOPs: 2 * 9 * Cin * Cout per real output pixel (the padded border is overhead)
    _timed("conv_fwd", 18.0 * N * (Hp - 2) * (Wp - 2) * Cin * cout, lambda: call(
        "pd_conv2d_fwd", dt(x_pad), _p(x_pad), N, Hp - 2, Wp - 2, Cin, _p(w), ldw, cout, _p(bias),
        dt(bias) if bias is not None else 0, int(relu), _p(y), _stream()), (N, Hp - 2, Cin, cout))
    return y


def conv2d_dgrad(dy_pad, w, ldw, cin, relu_aux=None):
    N, Hp, Wp, Cout = dy_pad.shape
    dx = torch.empty((N, Hp, Wp, cin), dtype=dy_pad.dtype, device=dy_pad.device)
    _timed("conv_dgrad", 18.0 * N * (Hp - 2) * (Wp - 2) * cin * Cout, lambda: call(
        "pd_conv2d_dgrad", dt(dy_pad), _p(dy_pad), N, Hp - 2, Wp - 2, Cout, _p(w), ldw, cin, _p(relu_aux), _p(dx),
        _stream()), (N, Hp - 2, cin, Cout))
    return dx


def conv2d_wgrad(x_pad, dy_pad, dw, lddw, accumulate=False, split_k=0):
    N, Hp, Wp, Cin = x_pad.shape
    Cout = dy_pad.shape[3]
    assert dw.dtype == torch.float32
    if _DETERMINISTIC and split_k == 0:
        split_k = 1
    _timed("conv_wgrad", 18.0 * N * (Hp - 2) * (Wp - 2) * Cin * Cout, lambda: call(
        "pd_conv2d_wgrad", dt(x_pad), _p(x_pad), _p(dy_pad), N, Hp - 2, Wp - 2, Cin, Cout, _p(dw), lddw,
        int(accumulate), int(split_k), _stream()), (N, Hp - 2, Cin, Cout))
    return dw


def gemm_poll_error():
    code = ctypes.c_int(0)
    call("pd_gemm_poll_error", ctypes.byref(code))
    return code.value


# --------------------------------------------------------------------------- #
# criteria and sequence utilities
# --------------------------------------------------------------------------- #
def softmax_ce_fwd(logits, target, smoothing, padding_idx, scale):
    """Returns (loss scalar fp32 tensor, lse[rows], row_loss[rows])."""
    _cuda(logits, target)
    rows, C = logits.shape
    row_loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    loss = torch.empty((), dtype=torch.float32, device=logits.device)
    call("pd_softmax_ce_fwd", _p(logits), dt(logits), _p(target), rows, C, float(smoothing), int(padding_idx),
         float(scale), _p(row_loss), _p(lse), _p(loss), _stream())
    return loss, lse, row_loss


def softmax_ce_bwd(logits, target, lse, smoothing, padding_idx, upstream, gscale):
    rows, C = logits.shape
    dlogits = torch.empty_like(logits)
    call("pd_softmax_ce_bwd", _p(logits), dt(logits), _p(target), _p(lse), rows, C, float(smoothing),
         int(padding_idx), _p(upstream), float(gscale), _p(dlogits), _stream())
    return dlogits


def revert_varlen(x, lengths):
    """x: [T,B,...] contiguous; lengths: int64 [B] on the same device."""
    _cuda(x, lengths)
    x = x if x.is_contiguous() else x.contiguous()
    T, B = x.shape[0], x.shape[1]
    out = torch.empty_like(x)
    fbytes = (x.numel() // (T * B)) * x.element_size()
    call("pd_revert_varlen", _p(x), _p(out), _p(lengths), T, B, fbytes, _stream())
    return out


def length_mask(lengths, T, dtype):
    _cuda(lengths)
    B = lengths.shape[0]
    out = torch.empty((T, B), dtype=dtype, device=lengths.device)
    code = 2 if dtype == torch.uint8 else _DT[dtype]
    call("pd_length_mask", _p(lengths), T, B, _p(out), code, _stream())
    return out


def mul_rows(x, mask):
    """y[r,:] = x[r,:] * mask[r]; x: [..., F] contiguous, mask: x.shape[:-1] in x's dtype."""
    _cuda(x, mask)
    F = x.shape[-1]
    y = torch.empty_like(x)
    call("pd_mul_rows", _p(x), _p(mask), _p(y), x.numel() // F, F, dt(x), _stream())
    return y


def embedding_fwd(ids, table):
    _cuda(ids, table)
    vocab, D = table.shape
    out = torch.empty(tuple(ids.shape) + (D,), dtype=table.dtype, device=table.device)
    call("pd_embedding_fwd", _p(ids), _p(table), ids.numel(), D, vocab, _p(out), dt(table), _stream())
    return out


def embedding_bwd(ids, dy, dtable, padding_idx):
    vocab, D = dtable.shape
    call("pd_embedding_bwd", _p(ids), _p(dy), ids.numel(), D, vocab, int(padding_idx), _p(dtable), dt(dy), _stream())
    return dtable


# --------------------------------------------------------------------------- #
# LSTM time loops
# --------------------------------------------------------------------------- #
_LSTM_STREAMS = {}
# The backward recurrence of a batch of 64..128 rows runs as two launches, the halves of the batch side by side on two
# streams (64 CTAs each at H = 1024; 0.74 -> 0.60 ms for 50 steps x 128 rows: each half hides the other's waits).  The
# forward recurrence stays one launch: its grid is 128 CTAs, two of them only fit with a shallower stage ring, and
# that costs more than the overlap gains (0.48 -> 0.53 ms measured).  PD_LSTM_SPLIT=0 switches the split off.
_LSTM_SPLIT = os.environ.get("PD_LSTM_SPLIT", "1") != "0"


def _lstm_halves(B, dtype):
    """The batch rows of the two launches, or None when the recurrence runs as one launch."""
    if not _LSTM_SPLIT or dtype != torch.bfloat16 or B < 64 or B > 128 or B % 2:
        return None
    return ((0, B // 2), (B // 2, B // 2))


def _lstm_side_streams(dev):
    st = _LSTM_STREAMS.get(dev.index)
    if st is None:
        st = _LSTM_STREAMS[dev.index] = (torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev))
    return st


def _run_halves(dev, launch):
    """launch(i, b0, Bh) on one of two side streams per half, ordered after the current stream; the current stream
    then waits for both.  Returns False if a launch declined (nothing may have been enqueued for that half)."""
    cur = torch.cuda.current_stream(dev)
    ok = True
    streams = _lstm_side_streams(dev)
    for i, st in enumerate(streams):
        st.wait_stream(cur)
        with torch.cuda.stream(st):
            ok = launch(i) and ok
        if not ok:
            break
    for st in streams:
        cur.wait_stream(st)
    return ok


def lstm_fwd(gx, w_hh, b_hh, T, B, H):
    """gx: [T*B, 4H] input projections (+ b_ih).  Returns (y [T,B,H], act [T,B,4H], c_all [T,B,H] fp32)."""
    _cuda(gx, w_hh)
    dev, dtype = gx.device, gx.dtype
    y = torch.empty((T, B, H), dtype=dtype, device=dev)
    act = torch.empty((T, B, 4 * H), dtype=dtype, device=dev)
    c_all = torch.empty((T, B, H), dtype=torch.float32, device=dev)
    gh_ws = torch.empty((B, 4 * H), dtype=torch.float32, device=dev)
    _timed("lstm_fwd", 2.0 * max(T - 1, 0) * B * 4 * H * H, lambda: call(
        "pd_lstm_fwd", dt(gx), _p(gx), _p(w_hh), _p(b_hh), T, B, H, _p(y), _p(act), _p(c_all), _p(gh_ws), _stream()),
        (T, B, H))
    return y, act, c_all


def lstm_bwd(dy, w_hh, act, c_all):
    """dy: [T,B,H] contiguous.  Returns dgates [T,B,4H] (gate pre-activation gradients)."""
    T, B, H = dy.shape
    dgates = torch.empty((T, B, 4 * H), dtype=dy.dtype, device=dy.device)
    dh_ws = torch.empty((B, H), dtype=torch.float32, device=dy.device)
    dc_ws = torch.empty((B, H), dtype=torch.float32, device=dy.device)
    halves = _lstm_halves(B, dy.dtype)
    if halves is not None:
        done = _timed("lstm_bwd", 2.0 * max(T - 1, 0) * B * 4 * H * H, lambda: _run_halves(dy.device, lambda i: _lib.call_or_decline(
            "pd_lstm_bwd_rows", dt(dy), _p(dy), _p(w_hh), _p(act), _p(c_all), T, B, halves[i][0], halves[i][1], H,
            _p(dgates), _p(dh_ws[halves[i][0]:]), _p(dc_ws[halves[i][0]:]), _stream())), (T, B, H))
        if done:
            return dgates
    _timed("lstm_bwd", 2.0 * max(T - 1, 0) * B * 4 * H * H, lambda: call(
        "pd_lstm_bwd", dt(dy), _p(dy), _p(w_hh), _p(act), _p(c_all), T, B, H, _p(dgates), _p(dh_ws), _p(dc_ws),
        _stream()), (T, B, H))
    return dgates


# --------------------------------------------------------------------------- #
# causal self-attention (transformer stages)
# --------------------------------------------------------------------------- #
def sdpa_causal_supported(qkv, heads):
    """Whether pd_sdpa_causal_fwd takes this projection output: bf16, head size 64, T a multiple of 128 up to 2048."""
    if qkv.dim() != 3 or qkv.dtype != torch.bfloat16 or not qkv.is_cuda:
        return False
    B, T, C3 = qkv.shape
    return C3 % (3 * heads) == 0 and C3 // (3 * heads) == 64 and T % 128 == 0 and 128 <= T <= 2048


def sdpa_causal_fwd(qkv, heads):
    """qkv [B, T, 3 * H * 64] contiguous bf16 -> (out [B, T, H * 64], probs [B * H, T, T])."""
    _cuda(qkv)
    B, T, C3 = qkv.shape
    C = C3 // 3
    d = C // heads
    out = torch.empty((B, T, C), dtype=qkv.dtype, device=qkv.device)
    probs = torch.empty((B * heads, T, T), dtype=qkv.dtype, device=qkv.device)
    _timed("sdpa_fwd", 2.0 * B * heads * T * T * d, lambda: call(
        "pd_sdpa_causal_fwd", dt(qkv), _p(qkv), B, T, heads, d, 1.0 / (d ** 0.5), _p(out), _p(probs), _stream()),
        (B, heads, T))
    return out, probs


def sdpa_causal_bwd(qkv, probs, dout, heads):
    """Gradient of sdpa_causal_fwd with respect to qkv."""
    B, T, C3 = qkv.shape
    d = C3 // 3 // heads
    dqkv = torch.empty_like(qkv)
    ws = torch.empty_like(probs)
    _timed("sdpa_bwd", 5.0 * B * heads * T * T * d, lambda: call(
        "pd_sdpa_causal_bwd", dt(qkv), _p(qkv), _p(probs), _p(dout), B, T, heads, d, 1.0 / (d ** 0.5), _p(dqkv), _p(ws),
        _stream()), (B, heads, T))
    return dqkv


# --------------------------------------------------------------------------- #
# additive attention
# --------------------------------------------------------------------------- #
def attn_fwd(pq, pk, keys_tbn, v, nb, ctx_len):
    """pq [b,tq,n], pk [b,tk,n] contiguous; keys_tbn [tk,b,nk] (sequence first, contiguous); v fp32 [n].
    Returns (probs [b,tq,tk], context [tq,b,nk])."""
    _cuda(pq, pk, keys_tbn, v, nb)
    b, tq, n = pq.shape
    tk, _, nk = keys_tbn.shape
    probs = torch.empty((b, tq, tk), dtype=pq.dtype, device=pq.device)
    context = torch.empty((tq, b, nk), dtype=pq.dtype, device=pq.device)
    call("pd_attn_bahdanau_fwd", dt(pq), _p(pq), _p(pk), _p(keys_tbn), nk, b * nk, _p(v), _p(nb), _p(ctx_len),
         b, tq, tk, n, nk, _p(probs), _p(context), nk, b * nk, _stream())
    return probs, context


def attn_bwd(pq, pk, keys_tbn, v, nb, probs, dcontext_tbn):
    """Returns (dpq, dpk, dkeys [tk,b,nk], dv fp32 [n], dnb fp32 [n])."""
    b, tq, n = pq.shape
    tk, _, nk = keys_tbn.shape
    dev = pq.device
    dpq, dpk = torch.empty_like(pq), torch.empty_like(pk)
    dkeys = torch.empty_like(keys_tbn)
    dv = torch.zeros(n, dtype=torch.float32, device=dev)
    dnb = torch.zeros(n, dtype=torch.float32, device=dev)
    ds_ws = torch.empty((b, tq, tk), dtype=torch.float32, device=dev)
    call("pd_attn_bahdanau_bwd", dt(pq), _p(pq), _p(pk), _p(keys_tbn), nk, b * nk, _p(v), _p(nb), _p(probs),
         _p(dcontext_tbn), nk, b * nk, b, tq, tk, n, nk, _p(dpq), _p(dpk), _p(dkeys), nk, b * nk, _p(dv), _p(dnb),
         _p(ds_ws), _stream())
    return dpq, dpk, dkeys, dv, dnb


# --------------------------------------------------------------------------- #
# batch norm, generic convolutions, ResNet pools
# --------------------------------------------------------------------------- #
def _bn_ws(device, C):
    return _workspace(device, _lib.load().pd_bn_workspace_bytes(C))


def bn_fwd(x_pad, gamma, beta, eps, momentum, relu, running_mean, running_var, res_pad=None):
    N, Hp, Wp, C = x_pad.shape
    dev = x_pad.device
    mean = torch.empty(C, dtype=torch.float32, device=dev)
    invstd = torch.empty(C, dtype=torch.float32, device=dev)
    y = torch.empty_like(x_pad)
    ws = _bn_ws(dev, C)
    call("pd_bn_fwd", dt(x_pad), _p(x_pad), _p(res_pad), N, Hp - 2, Wp - 2, C, _p(gamma), _p(beta), float(eps), float(momentum),
         int(relu), _p(mean), _p(invstd), _p(running_mean), _p(running_var), _p(y), _p(ws), ws.numel(), _stream())
    return y, mean, invstd


def bn_apply(x_pad, gamma, beta, mean, invstd, relu, res_pad=None):
    N, Hp, Wp, C = x_pad.shape
    y = torch.empty_like(x_pad)
    call("pd_bn_apply", dt(x_pad), _p(x_pad), _p(res_pad), N, Hp - 2, Wp - 2, C, _p(gamma), _p(beta), _p(mean), _p(invstd), int(relu),
         _p(y), _stream())
    return y


def bn_bwd(x_pad, dy_pad, y_pad, gamma, mean, invstd, dgamma, dbeta, accumulate, want_dres=False):
    N, Hp, Wp, C = x_pad.shape
    dev = x_pad.device
    dx = torch.empty_like(x_pad)
    dres = torch.empty_like(x_pad) if want_dres else None
    sums = torch.empty(2 * C, dtype=torch.float32, device=dev)
    ws = _bn_ws(dev, C)
    call("pd_bn_bwd", dt(x_pad), _p(x_pad), _p(dy_pad), _p(y_pad), N, Hp - 2, Wp - 2, C, _p(gamma), _p(mean), _p(invstd),
         _p(dgamma), _p(dbeta), int(accumulate), _p(dx), _p(dres), _p(sums), _p(ws), ws.numel(), _stream())
    return (dx, dres) if want_dres else dx


def im2col(x, kh, kw, stride, pad, kpad, dtype):
    """Any-stride [N,C,H,W] -> ([N*Ho*Wo, kpad] patch matrix, Ho, Wo)."""
    N, C, H, W = x.shape
    Ho, Wo = (H + 2 * pad - kh) // stride + 1, (W + 2 * pad - kw) // stride + 1
    out = torch.empty((N * Ho * Wo, kpad), dtype=dtype, device=x.device)
    sN, sC, sH, sW = x.stride()
    call("pd_im2col", _p(x), dt(x), sN, sC, sH, sW, N, C, H, W, kh, kw, stride, pad, Ho, Wo, kpad, _p(out), _DT[dtype],
         _stream())
    return out, Ho, Wo


def col2im_pnhwc(dcol, N, C, H, W, kh, kw, stride, pad, Ho, Wo):
    dx = torch.empty((N, H + 2, W + 2, C), dtype=dcol.dtype, device=dcol.device)
    call("pd_col2im_pnhwc", _p(dcol), N, C, H, W, kh, kw, stride, pad, Ho, Wo, dcol.shape[1], _p(dx), dt(dcol), _stream())
    return dx


def maxpool3s2_fwd(x_pad, want_argmax=True):
    """Returns (y_pad, argmax): argmax [N,Ho,Wo,C] uint8 = position r*3+s of each window's first maximum."""
    N, Hp, Wp, C = x_pad.shape
    H, W = Hp - 2, Wp - 2
    Ho, Wo = (H - 1) // 2 + 1, (W - 1) // 2 + 1
    y = torch.empty((N, Ho + 2, Wo + 2, C), dtype=x_pad.dtype, device=x_pad.device)
    amax = torch.empty((N, Ho, Wo, C), dtype=torch.uint8, device=x_pad.device) if want_argmax else None
    call("pd_maxpool3s2_fwd", _p(x_pad), N, C, H, W, _p(y), _p(amax), dt(x_pad), _stream())
    return y, amax


def maxpool3s2_bwd(amax, dy_pad, H, W):
    N, _, _, C = dy_pad.shape
    dx = torch.empty((N, H + 2, W + 2, C), dtype=dy_pad.dtype, device=dy_pad.device)
    call("pd_maxpool3s2_bwd", _p(amax), _p(dy_pad), N, C, H, W, _p(dx), dt(dy_pad), _stream())
    return dx


def avgpool_fwd(x_pad):
    N, Hp, Wp, C = x_pad.shape
    y = torch.empty((N, C, 1, 1), dtype=x_pad.dtype, device=x_pad.device)
    call("pd_avgpool_fwd", _p(x_pad), N, C, Hp - 2, Wp - 2, _p(y), dt(x_pad), _stream())
    return y


def avgpool_bwd(dy, N, C, H, W):
    dx = torch.empty((N, H + 2, W + 2, C), dtype=dy.dtype, device=dy.device)
    call("pd_avgpool_bwd", _p(dy), N, C, H, W, _p(dx), dt(dy), _stream())
    return dx


# --------------------------------------------------------------------------- #
# layer norm, GELU (transformer stages)
# --------------------------------------------------------------------------- #
def layernorm_fwd(x2d, gamma, beta, eps):
    """x2d: [rows, C] contiguous.  Returns (y, mean fp32 [rows], rstd fp32 [rows])."""
    _cuda(x2d, gamma, beta)
    rows, C = x2d.shape
    y = torch.empty_like(x2d)
    mean = torch.empty(rows, dtype=torch.float32, device=x2d.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x2d.device)
    call("pd_layernorm_fwd", dt(x2d), _p(x2d), rows, C, _p(gamma), _p(beta), float(eps), _p(y), _p(mean), _p(rstd), _stream())
    return y, mean, rstd


def layernorm_bwd(x2d, dy2d, gamma, mean, rstd, dgamma, dbeta, accumulate):
    rows, C = x2d.shape
    dx = torch.empty_like(x2d)
    ws = _workspace(x2d.device, _lib.load().pd_layernorm_workspace_bytes(rows, C))
    call("pd_layernorm_bwd", dt(x2d), _p(x2d), _p(dy2d), _p(gamma), _p(mean), _p(rstd), rows, C, _p(dx), _p(dgamma), _p(dbeta),
         int(accumulate), _p(ws), ws.numel(), _stream())
    return dx


def gelu_fwd(x, tanh_form):
    _cuda(x)
    y = torch.empty_like(x)
    call("pd_gelu_fwd", dt(x), _p(x), _p(y), x.numel(), int(tanh_form), _stream())
    return y


def gelu_bwd(x, dy, tanh_form):
    dx = torch.empty_like(x)
    call("pd_gelu_bwd", dt(x), _p(x), _p(dy), _p(dx), x.numel(), int(tanh_form), _stream())
    return dx
