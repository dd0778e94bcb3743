"""B200-native replacements for the leaf torch.nn modules a stage is built from.

A stage module (user code in the reference's generated format, e.g.
runtime/image_classification/models/vgg16/gpus=8/stage0.py:7-71) stays
unmodified; `nativize()` swaps its leaf modules for the classes below, which
keep the parameter names and shapes (so state_dict keys and checkpoints
interchange) but run hand-written CUDA kernels through the C-ABI.  4-D
activations travel between native modules as zero-copy logical-NCHW views of
padded-NHWC buffers (see functional.nchw_view).

Weight gradients are written by the kernels straight into `param._pd_grad`
(fp32, same element order as the parameter), which the weight-stashing
optimizer maps onto its flat gradient arena; autograd therefore receives None
for the parameters of native modules.
"""
import itertools

import os

import torch
import torch.nn as nn

from . import functional as pf

_SEED_COUNTER = itertools.count(1)


# --------------------------------------------------------------------------- #
# gradient buffers
# --------------------------------------------------------------------------- #
def grad_buffer(param):
    """fp32 gradient buffer of a parameter (same logical shape and strides)."""
    g = getattr(param, "_pd_grad", None)
    if g is None:
        data = param.data
        span = 1 + sum((s - 1) * st for s, st in zip(data.shape, data.stride())) if data.numel() else 0
        if data.dim() >= 2:
            span = max(span, data.shape[0] * data.stride(0))     # whole rows, incl. row padding
        store = torch.zeros(span, dtype=torch.float32, device=data.device)
        g = store.as_strided(data.shape, data.stride())
        param._pd_grad = g
        param._pd_acc = False
        if param.dtype == torch.float32:
            param.grad = g
    return g


def _mark_native(*params):
    """Gradients of these parameters are written by the kernels, not by autograd."""
    for p in params:
        if p is not None:
            p._pd_native = True


def take_accumulate_flag(param):
    """False on the first gradient write after zero_grad (store), True afterwards (accumulate).  Called right
    before the kernel that writes the gradient is enqueued; a replicated stage listens here to learn how far the
    backward pass has come (StageRuntime's GradientAverager)."""
    acc = getattr(param, "_pd_acc", False)
    param._pd_acc = True
    hook = getattr(param, "_pd_grad_hook", None)
    if hook is not None:
        hook(param)
    return acc


def _dense2d(t, rows, cols):
    """[rows, cols] alias of a tensor whose storage is row-major with leading dim stride(0)."""
    return t.as_strided((rows, cols), (t.stride(0), 1), t.storage_offset())


# --------------------------------------------------------------------------- #
# Conv2d 3x3 / stride 1 / pad 1
# --------------------------------------------------------------------------- #
_SIDE_STREAMS = {}
# PD_BIAS_GRAD_STREAM=0 keeps the bias-gradient sums on the main stream (for timing comparisons)
_USE_SIDE_STREAM = os.environ.get("PD_BIAS_GRAD_STREAM", "1") != "0"


def _bias_grad_beside(dy_pad, colsum, accumulate):
    """Column sums of dy_pad into `colsum` on the device's second stream, ordered after the work queued on the current
    stream so far.  Returns the stream; the caller makes the current stream wait for it."""
    dev = dy_pad.device
    side = _SIDE_STREAMS.get(dev.index)
    if side is None:
        side = _SIDE_STREAMS[dev.index] = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        pf.relu_bwd_colsum(dy_pad, None, None, colsum, accumulate)
    return side


class _Conv3x3Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, fuse_relu, out_nchw):
        w = weight.detach()          # alias of the weight version that is current now
        b = bias.detach() if bias is not None else None
        N, Cin, H, W = x.shape
        Cout = w.shape[0]
        ctx.direct = (Cin % 64 == 0)
        ctx.fuse_relu = fuse_relu
        ctx.weight_param = weight
        ctx.bias_param = bias
        ctx.geom = (N, Cin, H, W, Cout)
        # x is the output of a fused conv+ReLU: this layer's data gradient can apply that ReLU's
        # mask in its epilogue and save the producer a pass over the gradient
        ctx.premask = bool(getattr(x, "_pd_relu_out", False)) and ctx.direct
        if ctx.direct:
            x_pad = pf.as_padded(x, w.dtype)
            y_pad = pf.conv2d_fwd(x_pad, w, w.stride(0), Cout, b, fuse_relu)
            ctx.x_saved = x_pad
        else:
            kpad = w.stride(0)
            col = pf.im2col3x3(x, kpad, w.dtype)
            y2d = pf.gemm_nt(col, _dense2d(w, Cout, kpad), bias=b, relu=fuse_relu, pad_hw=(H + 2, W + 2))
            y_pad = y2d.view(N, H + 2, W + 2, Cout)
            ctx.x_saved = col    # the patch matrix (a few hundred MB at most) is kept for the weight gradient
        ctx.y_pad = y_pad if fuse_relu else None
        if out_nchw:
            return pf.unpack_pnhwc(y_pad)
        return pf.nchw_view(y_pad, N, Cout, H, W)

    @staticmethod
    def backward(ctx, dy):
        N, Cin, H, W, Cout = ctx.geom
        wp, bp = ctx.weight_param, ctx.bias_param
        # The data gradient uses the weights loaded in the module now (the optimizer's
        # load_old_params ran just before), as autograd does in the reference, where the
        # saved tensor aliases the parameter storage.
        w = wp.detach()
        dy_pad = pf.as_padded(dy, w.dtype)
        side = None
        # ReLU mask and bias gradient in one pass over dy; if the consumer's backward already applied
        # this layer's mask (see ctx.premask), only the bias gradient is left to do
        if ctx.fuse_relu and getattr(dy, "_pd_premasked", False) and pf.padded_of(dy) is not None:
            dym = dy_pad
            if bp is not None and getattr(dy, "_pd_colsum", None) is not None:
                pf.colsum_finish(dy._pd_colsum, grad_buffer(bp), take_accumulate_flag(bp))
            elif bp is not None and ctx.direct and ctx.needs_input_grad[0] and _USE_SIDE_STREAM:
                # a read-only pass over dy (bound by HBM): it runs on a second stream beside the data-gradient
                # contraction (bound by the tensor pipe); the main stream joins it before the weight gradient
                side = _bias_grad_beside(dy_pad, grad_buffer(bp), take_accumulate_flag(bp))
            elif bp is not None:
                pf.relu_bwd_colsum(dy_pad, None, None, grad_buffer(bp), take_accumulate_flag(bp))
        elif ctx.fuse_relu:
            dym = torch.empty_like(dy_pad)
            if bp is not None:
                pf.relu_bwd_colsum(dy_pad, ctx.y_pad, dym, grad_buffer(bp), take_accumulate_flag(bp))
            else:
                pf.relu_bwd(dy_pad, ctx.y_pad, out=dym)
        else:
            dym = dy_pad
            if bp is not None:
                pf.relu_bwd_colsum(dy_pad, None, None, grad_buffer(bp), take_accumulate_flag(bp))
        gw = grad_buffer(wp)
        dx = None
        if ctx.direct:
            x_pad = ctx.x_saved
            if ctx.needs_input_grad[0]:
                dx_pad = pf.conv2d_dgrad(dym, w, w.stride(0), Cin, relu_aux=x_pad if ctx.premask else None)
                dx = pf.nchw_view(dx_pad, N, Cin, H, W)
                if ctx.premask:
                    dx._pd_premasked = True
            if side is not None:
                # before the weight's gradient is announced: a gradient bucket that closes on that announcement
                # orders its all-reduce after the main stream, which must already include the bias gradient
                torch.cuda.current_stream(dym.device).wait_stream(side)
            pf.conv2d_wgrad(x_pad, dym, gw, gw.stride(0), accumulate=take_accumulate_flag(wp))
        else:
            kpad = w.stride(0)
            pf.gemm_tn(dym.view(-1, Cout), ctx.x_saved, _dense2d(gw, Cout, kpad), accumulate=take_accumulate_flag(wp))
            if ctx.needs_input_grad[0]:
                raise NotImplementedError("input gradient of a convolution with Cin %% 64 != 0 is not implemented")
        return dx, None, None, None, None


class NativeConv2d(nn.Module):
    """3x3 / stride 1 / padding 1 convolution (optionally fused with the ReLU that follows it)."""

    def __init__(self, conv):
        super().__init__()
        self.in_channels, self.out_channels = conv.in_channels, conv.out_channels
        self.kernel_size, self.stride, self.padding = conv.kernel_size, conv.stride, conv.padding
        self.fuse_relu = False
        self.out_nchw = True
        w = conv.weight.data
        cout, cin = w.shape[0], w.shape[1]
        if cin % 64 == 0:
            # [Cout][r][s][Cin] storage, logical shape unchanged
            conv.weight.data = w.contiguous(memory_format=torch.channels_last)
        else:
            # im2col path: rows of kpad >= 9*Cin elements (multiple of 32), zero filled
            kpad = ((9 * cin + 31) // 32) * 32
            store = torch.zeros(cout * kpad, dtype=w.dtype, device=w.device)
            view = store.as_strided((cout, cin, 3, 3), (kpad, 1, 3 * cin, cin))
            view.copy_(w)
            conv.weight.data = view
        self.weight = conv.weight
        self.bias = conv.bias
        _mark_native(self.weight, self.bias)

    @staticmethod
    def supports(conv):
        return (isinstance(conv, nn.Conv2d) and conv.kernel_size == (3, 3) and conv.stride == (1, 1)
                and conv.padding == (1, 1) and conv.dilation == (1, 1) and conv.groups == 1
                and conv.padding_mode == "zeros" and conv.out_channels % 8 == 0
                and (conv.in_channels % 64 == 0 or conv.in_channels < 8))

    def forward(self, x):
        y = _Conv3x3Fn.apply(x, self.weight, self.bias, self.fuse_relu, self.out_nchw)
        if self.fuse_relu and not self.out_nchw:
            y._pd_relu_out = True      # consumers may fold this ReLU's mask into their data gradient
        return y

    def extra_repr(self):
        return "%d, %d, kernel_size=(3, 3), stride=(1, 1), padding=(1, 1), fuse_relu=%s" % (
            self.in_channels, self.out_channels, self.fuse_relu)



# --------------------------------------------------------------------------- #
# ResNet pieces: batch norm, 1x1 and patch-matrix convolutions, 3x3/2 max-pool, global average pool
# --------------------------------------------------------------------------- #
class _BatchNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, res, weight, bias, mod, fuse_relu, out_nchw):
        N, C, H, W = x.shape
        g, b = weight.detach(), bias.detach()
        x_pad = pf.as_padded(x, g.dtype)
        res_pad = pf.as_padded(res, g.dtype) if res is not None else None
        y_pad, mean, invstd = pf.bn_fwd(x_pad, g, b, mod.eps, mod.momentum if mod.momentum is not None else 0.1,
                                        fuse_relu, mod.running_mean, mod.running_var, res_pad)
        ctx.saved = (x_pad, y_pad if fuse_relu else None, mean, invstd)
        ctx.params = (weight, bias)
        ctx.geom = (N, C, H, W)
        ctx.has_res = res is not None
        return pf.unpack_pnhwc(y_pad) if out_nchw else pf.nchw_view(y_pad, N, C, H, W)

    @staticmethod
    def backward(ctx, dy):
        x_pad, y_pad, mean, invstd = ctx.saved
        weight, bias = ctx.params
        N, C, H, W = ctx.geom
        g = weight.detach()
        dy_pad = pf.as_padded(dy, g.dtype)
        acc = take_accumulate_flag(weight)
        take_accumulate_flag(bias)
        dres = None
        if ctx.has_res and ctx.needs_input_grad[1] and y_pad is not None:
            # the masked upstream gradient is the shortcut's gradient: written by the same pass
            dx_pad, dres_pad = pf.bn_bwd(x_pad, dy_pad, y_pad, g, mean, invstd, grad_buffer(weight), grad_buffer(bias),
                                         acc, want_dres=True)
            dres = pf.nchw_view(dres_pad, N, C, H, W)
        else:
            dx_pad = pf.bn_bwd(x_pad, dy_pad, y_pad, g, mean, invstd, grad_buffer(weight), grad_buffer(bias), acc)
            if ctx.has_res and ctx.needs_input_grad[1]:
                dres = pf.nchw_view(dy_pad, N, C, H, W)
        return pf.nchw_view(dx_pad, N, C, H, W), dres, None, None, None, None, None


class NativeBatchNorm2d(nn.Module):
    def __init__(self, bn):
        super().__init__()
        self.num_features, self.eps, self.momentum = bn.num_features, bn.eps, bn.momentum
        self.fuse_relu = False
        self.out_nchw = True
        self.weight, self.bias = bn.weight, bn.bias
        # statistics stay fp32 whatever the compute dtype (the reference keeps BN in fp32 under fp16 too,
        # runtime/runtime.py:229)
        self.register_buffer("running_mean", bn.running_mean.detach().float().clone())
        self.register_buffer("running_var", bn.running_var.detach().float().clone())
        # kept on the host: incrementing it every step would otherwise be one more (tiny) launch per layer
        self.register_buffer("num_batches_tracked", bn.num_batches_tracked.detach().cpu().clone())
        _mark_native(self.weight, self.bias)

    @staticmethod
    def supports(m):
        return (isinstance(m, nn.BatchNorm2d) and m.affine and m.track_running_stats and m.num_features % 8 == 0
                and m.num_features <= 2048)

    def forward(self, x, res=None):
        """res: optional tensor of x's shape that is added after the normalisation (before the fused ReLU)."""
        if self.training:
            self.num_batches_tracked.add_(1)
            return _BatchNormFn.apply(x, res, self.weight, self.bias, self, self.fuse_relu, self.out_nchw)
        N, C, H, W = x.shape
        invstd = torch.rsqrt(self.running_var + self.eps)
        y_pad = pf.bn_apply(pf.as_padded(x, self.weight.dtype), self.weight.detach(), self.bias.detach(),
                            self.running_mean, invstd, self.fuse_relu,
                            pf.as_padded(res, self.weight.dtype) if res is not None else None)
        return pf.unpack_pnhwc(y_pad) if self.out_nchw else pf.nchw_view(y_pad, N, C, H, W)


class _ForkFn(torch.autograd.Function):
    """Two aliases of one padded tensor; the two gradients are summed by one dense pass over the padded
    buffers (autograd's own accumulation would add strided views and lose the layout)."""

    @staticmethod
    def forward(ctx, x):
        ctx.geom = x.shape
        return x.view_as(x), x.view_as(x)

    @staticmethod
    def backward(ctx, d1, d2):
        if d1 is None or d2 is None:
            return d1 if d2 is None else d2
        p1, p2 = pf.padded_of(d1), pf.padded_of(d2)
        if p1 is None or p2 is None or p1.dtype != p2.dtype:
            return d1 + d2
        N, C, H, W = ctx.geom
        return pf.nchw_view(pf.add(p1, p2), N, C, H, W)


class NativeFork(nn.Module):
    """Inserted by nativize() where a padded result has two consumers (a residual block's input)."""

    def forward(self, x):
        if not (torch.is_grad_enabled() and x.requires_grad):
            return x, x
        return _ForkFn.apply(x)


def _dense_nhwc(t, dtype):
    """[N*H*W, C] dense matrix of a logical NCHW tensor of any strides (a 1x1 patch matrix)."""
    N, C, H, W = t.shape
    if t.dtype == dtype and t.stride() == (H * W * C, 1, W * C, C):
        return t.permute(0, 2, 3, 1).reshape(N * H * W, C)
    return pf.im2col(t, 1, 1, 1, 0, C, dtype)[0]


class _Conv1x1Fn(torch.autograd.Function):
    """1x1 / stride 1 convolution: a plain contraction over the padded pixel rows."""

    @staticmethod
    def forward(ctx, x, weight, bias, out_nchw):
        w = weight.detach()
        N, Cin, H, W = x.shape
        Cout = w.shape[0]
        x_pad = pf.as_padded(x, w.dtype)
        y2d = pf.gemm_nt(x_pad.view(-1, Cin), _dense2d(w, Cout, Cin), bias=bias.detach() if bias is not None else None,
                         pad_hw=(H + 2, W + 2))
        ctx.x_pad, ctx.params, ctx.geom = x_pad, (weight, bias), (N, Cin, H, W, Cout)
        y_pad = y2d.view(N, H + 2, W + 2, Cout)
        return pf.unpack_pnhwc(y_pad) if out_nchw else pf.nchw_view(y_pad, N, Cout, H, W)

    @staticmethod
    def backward(ctx, dy):
        weight, bias = ctx.params
        N, Cin, H, W, Cout = ctx.geom
        w = weight.detach()
        dy2d = pf.as_padded(dy, w.dtype).view(-1, Cout)
        gw = grad_buffer(weight)
        pf.gemm_tn(dy2d, ctx.x_pad.view(-1, Cin), _dense2d(gw, Cout, Cin), accumulate=take_accumulate_flag(weight))
        if bias is not None:
            pf.relu_bwd_colsum(dy2d, None, None, grad_buffer(bias), take_accumulate_flag(bias))
        dx = None
        if ctx.needs_input_grad[0]:
            dx_pad = pf.gemm_nn(dy2d, _dense2d(w, Cout, Cin)).view(N, H + 2, W + 2, Cin)
            dx = pf.nchw_view(dx_pad, N, Cin, H, W)
        return dx, None, None, None


class _ConvPatchFn(torch.autograd.Function):
    """Any other convolution (7x7 stride 2, 1x1 / 3x3 stride 2, ...): patch matrix + contraction."""

    @staticmethod
    def forward(ctx, x, weight, bias, geom):
        kh, kw, stride, pad = geom
        w = weight.detach()
        N, Cin, H, W = x.shape
        Cout, kpad = w.shape[0], w.stride(0)
        col, Ho, Wo = pf.im2col(x, kh, kw, stride, pad, kpad, w.dtype)
        y2d = pf.gemm_nt(col, _dense2d(w, Cout, kpad), bias=bias.detach() if bias is not None else None)
        ctx.col, ctx.params, ctx.geom = col, (weight, bias), (N, Cin, H, W, Cout, Ho, Wo, kh, kw, stride, pad, kpad)
        return y2d.view(N, Ho, Wo, Cout).permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        weight, bias = ctx.params
        N, Cin, H, W, Cout, Ho, Wo, kh, kw, stride, pad, kpad = ctx.geom
        w = weight.detach()
        dy2d = _dense_nhwc(dy, w.dtype)
        gw = grad_buffer(weight)
        pf.gemm_tn(dy2d, ctx.col, _dense2d(gw, Cout, kpad), accumulate=take_accumulate_flag(weight))
        if bias is not None:
            pf.relu_bwd_colsum(dy2d, None, None, grad_buffer(bias), take_accumulate_flag(bias))
        dx = None
        if ctx.needs_input_grad[0]:
            dcol = pf.gemm_nn(dy2d, _dense2d(w, Cout, kpad))
            dx = pf.nchw_view(pf.col2im_pnhwc(dcol, N, Cin, H, W, kh, kw, stride, pad, Ho, Wo), N, Cin, H, W)
        return dx, None, None, None


class NativeConvGeneric(nn.Module):
    """Conv2d with a square kernel, any stride / padding, groups = 1, dilation 1, that is not 3x3 / stride 1."""

    def __init__(self, conv):
        super().__init__()
        self.in_channels, self.out_channels = conv.in_channels, conv.out_channels
        self.kernel_size, self.stride, self.padding = conv.kernel_size, conv.stride, conv.padding
        self.out_nchw = True
        self.is_1x1 = conv.kernel_size == (1, 1) and conv.stride == (1, 1) and conv.padding == (0, 0) \
            and conv.in_channels % 8 == 0
        w = conv.weight.data
        cout, cin, kh, kw = w.shape
        if not self.is_1x1:
            K = kh * kw * cin
            kpad = K if K % 8 == 0 else ((K + 31) // 32) * 32
            store = torch.zeros(cout * kpad, dtype=w.dtype, device=w.device)
            view = store.as_strided((cout, cin, kh, kw), (kpad, 1, kw * cin, cin))
            view.copy_(w)
            conv.weight.data = view
        self.weight, self.bias = conv.weight, conv.bias
        _mark_native(self.weight, self.bias)

    @staticmethod
    def supports(m):
        return (isinstance(m, nn.Conv2d) and m.groups == 1 and m.dilation == (1, 1) and m.padding_mode == "zeros"
                and m.kernel_size[0] == m.kernel_size[1] and m.stride[0] == m.stride[1]
                and m.padding[0] == m.padding[1] and m.out_channels % 8 == 0 and not NativeConv2d.supports(m))

    def forward(self, x):
        if self.is_1x1:
            return _Conv1x1Fn.apply(x, self.weight, self.bias, self.out_nchw)
        return _ConvPatchFn.apply(x, self.weight, self.bias,
                                  (self.kernel_size[0], self.kernel_size[1], self.stride[0], self.padding[0]))


class _MaxPool3s2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_nchw):
        N, C, H, W = x.shape
        x_pad = pf.as_padded(x)
        y_pad, amax = pf.maxpool3s2_fwd(x_pad, want_argmax=ctx.needs_input_grad[0])
        ctx.amax, ctx.geom = amax, (N, C, H, W)
        Ho, Wo = y_pad.shape[1] - 2, y_pad.shape[2] - 2
        return pf.unpack_pnhwc(y_pad) if out_nchw else pf.nchw_view(y_pad, N, C, Ho, Wo)

    @staticmethod
    def backward(ctx, dy):
        N, C, H, W = ctx.geom
        return pf.nchw_view(pf.maxpool3s2_bwd(ctx.amax, pf.as_padded(dy), H, W), N, C, H, W), None


class NativeMaxPool3s2(nn.Module):
    def __init__(self):
        super().__init__()
        self.out_nchw = True

    @staticmethod
    def supports(m):
        def eq(v, k):
            return v == k or v == (k, k)
        return (isinstance(m, nn.MaxPool2d) and eq(m.kernel_size, 3) and eq(m.stride, 2) and eq(m.padding, 1)
                and eq(m.dilation, 1) and not m.ceil_mode and not m.return_indices)

    def forward(self, x):
        return _MaxPool3s2Fn.apply(x, self.out_nchw)


class _GlobalAvgPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        N, C, H, W = x.shape
        ctx.geom = (N, C, H, W)
        return pf.avgpool_fwd(pf.as_padded(x))

    @staticmethod
    def backward(ctx, dy):
        N, C, H, W = ctx.geom
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        return pf.nchw_view(pf.avgpool_bwd(dyc, N, C, H, W), N, C, H, W)


class NativeGlobalAvgPool(nn.Module):
    """AvgPool2d whose window is the whole feature map (AvgPool2d(7) on the 7x7 map of ResNet-50)."""

    def __init__(self, kernel):
        super().__init__()
        self.kernel = kernel

    @staticmethod
    def supports(m):
        k = m.kernel_size if isinstance(m, nn.AvgPool2d) else None
        return isinstance(m, nn.AvgPool2d) and (m.padding in (0, (0, 0))) and not m.ceil_mode and k is not None

    def forward(self, x):
        k = self.kernel if isinstance(self.kernel, tuple) else (self.kernel, self.kernel)
        if (x.shape[2], x.shape[3]) != k:
            raise pf._lib.PipedreamB200Error("NativeGlobalAvgPool: window %s does not cover the %dx%d map" % (
                k, x.shape[2], x.shape[3]))
        return _GlobalAvgPoolFn.apply(x)

# --------------------------------------------------------------------------- #
# ReLU / MaxPool / Dropout
# --------------------------------------------------------------------------- #
class _ReLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_nchw):
        if x.dim() == 4:
            N, C, H, W = x.shape
            y_pad = pf.relu(pf.as_padded(x))
            ctx.y = y_pad
            ctx.geom = (N, C, H, W)
            return pf.unpack_pnhwc(y_pad) if out_nchw else pf.nchw_view(y_pad, N, C, H, W)
        xc = x if x.is_contiguous() else x.contiguous()
        y = pf.relu(xc)
        ctx.y = y.detach()        # not the returned object itself (reference cycle through grad_fn)
        ctx.geom = None
        return y

    @staticmethod
    def backward(ctx, dy):
        if ctx.geom is not None:
            N, C, H, W = ctx.geom
            dx_pad = pf.relu_bwd(pf.as_padded(dy), ctx.y)
            return pf.nchw_view(dx_pad, N, C, H, W), None
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        return pf.relu_bwd(dyc, ctx.y), None


class NativeReLU(nn.Module):
    def __init__(self):
        super().__init__()
        self.out_nchw = True

    def forward(self, x):
        return _ReLUFn.apply(x, self.out_nchw)


class FusedAway(nn.Module):
    """Stands in for a module whose work was folded into the producer's epilogue."""

    def forward(self, x):
        return x


class _MaxPool2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_nchw):
        N, C, H, W = x.shape
        x_pad = pf.as_padded(x)
        ctx.x_pad = x_pad
        ctx.geom = (N, C, H, W)
        ctx.premask = bool(getattr(x, "_pd_relu_out", False))
        y = pf.maxpool2_fwd(x_pad, out_nchw)
        return y if out_nchw else pf.nchw_view(y, N, C, H // 2, W // 2)

    @staticmethod
    def backward(ctx, dy):
        N, C, H, W = ctx.geom
        dy_pad = pf.padded_of(dy)
        colsum = None
        if dy_pad is not None and ctx.premask and pf.maxpool2_bwd_colsum_ok(ctx.x_pad):
            # the producer is a fused conv+ReLU: its bias gradient (column sums of dx) comes out of the same pass
            dx_pad, colsum = pf.maxpool2_bwd_colsum(ctx.x_pad, dy_pad, True)
        elif dy_pad is not None:
            dx_pad = pf.maxpool2_bwd(ctx.x_pad, dy_pad, False, ctx.premask)
        else:
            dyc = dy if dy.is_contiguous() else dy.contiguous()
            dx_pad = pf.maxpool2_bwd(ctx.x_pad, dyc, True, ctx.premask)
        dx = pf.nchw_view(dx_pad, N, C, H, W)
        if ctx.premask:
            dx._pd_premasked = True
        if colsum is not None:
            dx._pd_colsum = colsum
        return dx, None


class NativeMaxPool2d(nn.Module):
    """2x2 / stride 2 max-pool."""

    def __init__(self):
        super().__init__()
        self.out_nchw = True

    @staticmethod
    def supports(m):
        def two(v):
            return v == 2 or v == (2, 2)
        return (isinstance(m, nn.MaxPool2d) and two(m.kernel_size) and two(m.stride) and m.padding in (0, (0, 0))
                and m.dilation in (1, (1, 1)) and not m.ceil_mode and not m.return_indices)

    def forward(self, x):
        if x.shape[2] % 2 or x.shape[3] % 2:
            raise pf._lib.PipedreamB200Error("NativeMaxPool2d needs even H and W")
        return _MaxPool2Fn.apply(x, self.out_nchw)


class _DropoutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed, offset):
        xc = x if x.is_contiguous() else x.contiguous()
        y, mask = pf.dropout_fwd(xc, p, seed, offset)
        ctx.mask, ctx.p = mask, p
        return y

    @staticmethod
    def backward(ctx, dy):
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        return pf.dropout_bwd(dyc, ctx.mask, ctx.p), None, None, None


class NativeDropout(nn.Module):
    def __init__(self, p):
        super().__init__()
        self.p = float(p)
        self.seed = next(_SEED_COUNTER) * 7919 + torch.initial_seed() % (1 << 31)
        self.offset = 0

    def forward(self, x):
        if not self.training or self.p == 0.0:
            return x
        off = self.offset
        self.offset += x.numel()
        return _DropoutFn.apply(x, self.p, self.seed, off)


# --------------------------------------------------------------------------- #
# LayerNorm, GELU (transformer stages)
# --------------------------------------------------------------------------- #
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        g, b = weight.detach(), bias.detach()
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != g.dtype:
            x2 = pf.convert(x2.contiguous(), g.dtype)
        elif not x2.is_contiguous():
            x2 = x2.contiguous()
        y, mean, rstd = pf.layernorm_fwd(x2, g, b, eps)
        ctx.saved = (x2, mean, rstd)
        ctx.params = (weight, bias)
        ctx.in_dtype = x.dtype
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, mean, rstd = ctx.saved
        weight, bias = ctx.params
        g = weight.detach()
        dy2 = dy.reshape(x2.shape)
        if dy2.dtype != g.dtype:
            dy2 = pf.convert(dy2.contiguous(), g.dtype)
        elif not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        acc = take_accumulate_flag(weight)
        take_accumulate_flag(bias)
        dx = pf.layernorm_bwd(x2, dy2, g, mean, rstd, grad_buffer(weight), grad_buffer(bias), acc)
        dx = dx.view(dy.shape)
        return (dx if dx.dtype == ctx.in_dtype else dx.to(ctx.in_dtype)), None, None, None


class NativeLayerNorm(nn.Module):
    def __init__(self, ln):
        super().__init__()
        self.normalized_shape, self.eps = ln.normalized_shape, ln.eps
        self.weight, self.bias = ln.weight, ln.bias
        _mark_native(self.weight, self.bias)

    @staticmethod
    def supports(m):
        return (isinstance(m, nn.LayerNorm) and m.elementwise_affine and m.bias is not None
                and len(m.normalized_shape) == 1 and m.normalized_shape[0] <= 1024)

    def forward(self, x):
        return _LayerNormFn.apply(x, self.weight, self.bias, self.eps)


class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tanh_form):
        xc = x if x.is_contiguous() else x.contiguous()
        ctx.x, ctx.tanh_form = xc, tanh_form
        return pf.gelu_fwd(xc, tanh_form)

    @staticmethod
    def backward(ctx, dy):
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        return pf.gelu_bwd(ctx.x, dyc, ctx.tanh_form), None


class NativeGELU(nn.Module):
    def __init__(self, approximate="none"):
        super().__init__()
        self.approximate = approximate

    def forward(self, x):
        return _GeluFn.apply(x, self.approximate == "tanh")


# --------------------------------------------------------------------------- #
# Linear
# --------------------------------------------------------------------------- #
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, fuse_relu):
        w = weight.detach()
        b = bias.detach() if bias is not None else None
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != w.dtype:
            x2 = pf.convert(x2.contiguous(), w.dtype)
        elif not x2.is_contiguous():
            x2 = x2.contiguous()
        y = pf.gemm_nt(x2, w, bias=b, relu=fuse_relu)
        ctx.x2, ctx.y = x2, (y if fuse_relu else None)
        ctx.weight_param, ctx.bias_param, ctx.fuse_relu, ctx.lead = weight, bias, fuse_relu, lead
        ctx.x_dtype = x.dtype
        return y.view(*lead, w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        wp, bp = ctx.weight_param, ctx.bias_param
        w, x2 = wp.detach(), ctx.x2     # weights loaded at backward time (see _Conv3x3Fn.backward)
        Nout = w.shape[0]
        dy2 = dy.reshape(-1, Nout)
        if dy2.dtype != w.dtype:
            dy2 = pf.convert(dy2.contiguous(), w.dtype)
        elif not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.fuse_relu:
            dym = torch.empty_like(dy2)
            if bp is not None:
                pf.relu_bwd_colsum(dy2, ctx.y, dym, grad_buffer(bp), take_accumulate_flag(bp))
            else:
                pf.relu_bwd(dy2, ctx.y, out=dym)
        else:
            dym = dy2
            if bp is not None:
                pf.relu_bwd_colsum(dy2, None, None, grad_buffer(bp), take_accumulate_flag(bp))
        gw = grad_buffer(wp)
        pf.gemm_tn(dym, x2, gw, accumulate=take_accumulate_flag(wp))
        dx = None
        if ctx.needs_input_grad[0]:
            dx = pf.gemm_nn(dym, w).view(*ctx.lead, w.shape[1])
            if dx.dtype != ctx.x_dtype:
                dx = pf.convert(dx, ctx.x_dtype)
        return dx, None, None, None


class NativeLinear(nn.Module):
    def __init__(self, lin):
        super().__init__()
        self.in_features, self.out_features = lin.in_features, lin.out_features
        self.fuse_relu = False
        self.weight = lin.weight
        self.bias = lin.bias
        _mark_native(self.weight, self.bias)

    @staticmethod
    def supports(m):
        return isinstance(m, nn.Linear) and m.in_features % 8 == 0 and m.out_features % 8 == 0

    def forward(self, x):
        return _LinearFn.apply(x, self.weight, self.bias, self.fuse_relu)

    def extra_repr(self):
        return "in_features=%d, out_features=%d, fuse_relu=%s" % (self.in_features, self.out_features, self.fuse_relu)



# --------------------------------------------------------------------------- #
# LSTM (one layer, one direction, sequence first)
# --------------------------------------------------------------------------- #
class _CausalAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, heads):
        qkv = qkv if qkv.is_contiguous() else qkv.contiguous()
        out, probs = pf.sdpa_causal_fwd(qkv, heads)
        ctx.heads = heads
        ctx.save_for_backward(qkv, probs)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, probs = ctx.saved_tensors
        dout = dout if dout.is_contiguous() else dout.contiguous()
        return pf.sdpa_causal_bwd(qkv, probs, dout, ctx.heads), None


class NativeCausalAttentionCore(nn.Module):
    """The attention core of a GPT block (gpt_blocks.CausalAttentionCore) on the tensor cores: batched tcgen05
    contractions for Q K^T, P V and their gradients, row kernels for the causal softmax (csrc/pd_sdpa.cu).  Shapes the
    kernels are not written for (head size other than 64, sequence not a multiple of 128, fp32 - the parity
    configuration) run the original module, torch's scaled_dot_product_attention; `native_calls` counts the others."""

    def __init__(self, core):
        super().__init__()
        self.heads = core.heads
        self.reference = core
        self.native_calls = 0

    @staticmethod
    def supports(m):
        return type(m).__name__ == "CausalAttentionCore" and hasattr(m, "heads")

    def forward(self, qkv):
        if pf.sdpa_causal_supported(qkv, self.heads):
            self.native_calls += 1
            return _CausalAttnFn.apply(qkv, self.heads)
        return self.reference(qkv)


class _LSTMFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_ih, w_hh, b_ih, b_hh):
        wi, wh = w_ih.detach(), w_hh.detach()
        T, B, I = x.shape
        H = wh.shape[1]
        x2 = x.reshape(T * B, I)
        if x2.dtype != wi.dtype:
            x2 = pf.convert(x2.contiguous(), wi.dtype)
        elif not x2.is_contiguous():
            x2 = x2.contiguous()
        gx = pf.gemm_nt(x2, wi, bias=b_ih.detach() if b_ih is not None else None)
        y, act, c_all = pf.lstm_fwd(gx, wh, b_hh.detach() if b_hh is not None else None, T, B, H)
        # an output kept on ctx must be a different tensor object than the one returned: the returned one gets
        # this node as its grad_fn, and node -> tensor -> node is a cycle no collector can see (it leaks the step)
        ctx.saved = (x2, y.detach(), act, c_all)
        ctx.params = (w_ih, w_hh, b_ih, b_hh)
        ctx.geom = (T, B, I, H)
        ctx.x_dtype = x.dtype
        ctx.c_last = c_all[T - 1]
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, y, act, c_all = ctx.saved
        w_ih, w_hh, b_ih, b_hh = ctx.params
        T, B, I, H = ctx.geom
        wi, wh = w_ih.detach(), w_hh.detach()      # weights loaded at backward time
        dyc = dy
        if dyc.dtype != wi.dtype:
            dyc = pf.convert(dyc.contiguous(), wi.dtype)
        elif not dyc.is_contiguous():
            dyc = dyc.contiguous()
        dgates = pf.lstm_bwd(dyc, wh, act, c_all)
        dg2 = dgates.view(T * B, 4 * H)
        pf.gemm_tn(dg2, x2, grad_buffer(w_ih), accumulate=take_accumulate_flag(w_ih))
        ghh = grad_buffer(w_hh)
        acc_hh = take_accumulate_flag(w_hh)
        if T > 1:
            pf.gemm_tn(dg2[B:], y.view(T * B, H)[:(T - 1) * B], ghh, accumulate=acc_hh)
        elif not acc_hh:
            ghh.zero_()
        for bp in (b_ih, b_hh):
            if bp is not None:
                pf.relu_bwd_colsum(dg2, None, None, grad_buffer(bp), take_accumulate_flag(bp))
        dx = None
        if ctx.needs_input_grad[0]:
            dx = pf.gemm_nn(dg2, wi).view(T, B, I)
            if dx.dtype != ctx.x_dtype:
                dx = pf.convert(dx, ctx.x_dtype)
        return dx, None, None, None, None


class NativeLSTM(nn.Module):
    """torch.nn.LSTM(input_size, hidden_size): one layer, one direction, [T,B,*] input, zero initial state."""

    def __init__(self, lstm):
        super().__init__()
        self.input_size, self.hidden_size = lstm.input_size, lstm.hidden_size
        self.weight_ih_l0 = lstm.weight_ih_l0
        self.weight_hh_l0 = lstm.weight_hh_l0
        self.bias_ih_l0 = lstm.bias_ih_l0 if lstm.bias else None
        self.bias_hh_l0 = lstm.bias_hh_l0 if lstm.bias else None
        _mark_native(self.weight_ih_l0, self.weight_hh_l0, self.bias_ih_l0, self.bias_hh_l0)

    @staticmethod
    def supports(m):
        return (isinstance(m, nn.LSTM) and m.num_layers == 1 and not m.bidirectional and not m.batch_first
                and getattr(m, "proj_size", 0) == 0 and m.input_size % 8 == 0 and m.hidden_size % 8 == 0)

    def forward(self, x, hx=None):
        if hx is not None:
            raise NotImplementedError("NativeLSTM starts from a zero state (the stage modules pass None)")
        y = _LSTMFn.apply(x, self.weight_ih_l0, self.weight_hh_l0, self.bias_ih_l0, self.bias_hh_l0)
        with torch.no_grad():
            h_n = y.detach()[-1:]
        return y, (h_n, None)

    def extra_repr(self):
        return "%d, %d" % (self.input_size, self.hidden_size)


class _RevertVarlenFn(torch.autograd.Function):
    """Per-sequence time reversal (its own inverse, so also its own gradient):
    runtime/translation/seq2seq/models/encoder.py:13-21."""

    @staticmethod
    def forward(ctx, x, lengths):
        ctx.lengths = lengths
        return pf.revert_varlen(x, lengths)

    @staticmethod
    def backward(ctx, dy):
        return pf.revert_varlen(dy, ctx.lengths), None


class _MaskRowsFn(torch.autograd.Function):
    """y[t,b,:] = x[t,b,:] * (t < len[b])."""

    @staticmethod
    def forward(ctx, x, lengths):
        T, B = x.shape[0], x.shape[1]
        mask = pf.length_mask(lengths, T, x.dtype)
        ctx.mask = mask
        return pf.mul_rows(x if x.is_contiguous() else x.contiguous(), mask)

    @staticmethod
    def backward(ctx, dy):
        return pf.mul_rows(dy if dy.is_contiguous() else dy.contiguous(), ctx.mask), None


class NativeEmuBidirLSTM(nn.Module):
    """Bidirectional first encoder layer built from two one-direction LSTMs, the second one run on the
    per-sequence time-reversed input (runtime/translation/seq2seq/models/encoder.py:25-64, the path taken
    for batches of at most 128).  Keeps the attribute layout `bidir`, `layer1`, `layer2` of the module it
    replaces, so parameter names do not change."""

    def __init__(self, emu):
        super().__init__()
        self.bidir = emu.bidir                 # owns the parameters under their bidirectional names
        self.layer1 = NativeLSTM(emu.layer1)
        self.layer2 = NativeLSTM(emu.layer2)

    @staticmethod
    def supports(m):
        return (type(m).__name__ == "EmuBidirLSTM" and all(hasattr(m, a) for a in ("bidir", "layer1", "layer2"))
                and NativeLSTM.supports(m.layer1) and NativeLSTM.supports(m.layer2))

    def forward(self, input, lengths):
        lengths = lengths.to(device=input.device, dtype=torch.int64)
        rev_in = _RevertVarlenFn.apply(input, lengths)
        out_rev = _RevertVarlenFn.apply(self.layer2(rev_in)[0], lengths)
        out_fwd = _MaskRowsFn.apply(self.layer1(input)[0], lengths)
        return torch.cat([out_fwd, out_rev], dim=2)


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, padding_idx):
        w = weight.detach()
        idc = ids if ids.is_contiguous() else ids.contiguous()
        ctx.ids, ctx.weight_param, ctx.padding_idx = idc, weight, padding_idx
        return pf.embedding_fwd(idc, w)

    @staticmethod
    def backward(ctx, dy):
        wp = ctx.weight_param
        g = grad_buffer(wp)
        if not take_accumulate_flag(wp):
            g.zero_()
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        pf.embedding_bwd(ctx.ids, dyc, g, ctx.padding_idx if ctx.padding_idx is not None else -1)
        return None, None, None


class NativeEmbedding(nn.Module):
    def __init__(self, emb):
        super().__init__()
        self.num_embeddings, self.embedding_dim, self.padding_idx = emb.num_embeddings, emb.embedding_dim, emb.padding_idx
        self.weight = emb.weight
        _mark_native(self.weight)

    @staticmethod
    def supports(m):
        return (isinstance(m, nn.Embedding) and m.max_norm is None and not m.scale_grad_by_freq and not m.sparse
                and m.embedding_dim % 8 == 0)

    def forward(self, ids):
        return _EmbeddingFn.apply(ids, self.weight, self.padding_idx)


# --------------------------------------------------------------------------- #
# additive attention
# --------------------------------------------------------------------------- #
class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pq, pk, keys, v, nb, ctx_len):
        nbd = nb.detach()
        if nbd.dtype != pq.dtype:
            nbd = nbd.to(pq.dtype)
        vf = v.detach().float().contiguous()
        keys_c = keys if keys.is_contiguous() else keys.contiguous()
        probs, context = pf.attn_fwd(pq.contiguous(), pk.contiguous(), keys_c, vf, nbd, ctx_len)
        ctx.saved = (pq, pk, keys_c, vf, nbd, probs.detach())   # not the returned object (cycle through grad_fn)
        ctx.v_dtype, ctx.nb_dtype = v.dtype, nb.dtype
        ctx.mark_non_differentiable(probs)
        return context, probs

    @staticmethod
    def backward(ctx, dcontext, _dprobs):
        pq, pk, keys_c, vf, nbd, probs = ctx.saved
        dc = dcontext if dcontext.is_contiguous() else dcontext.contiguous()
        dpq, dpk, dkeys, dv, dnb = pf.attn_bwd(pq.contiguous(), pk.contiguous(), keys_c, vf, nbd, probs, dc)
        return dpq, dpk, dkeys, dv.to(ctx.v_dtype), dnb.to(ctx.nb_dtype), None


class NativeBahdanauAttention(nn.Module):
    """Normalised additive attention over sequence-first tensors (query [t_q,b,n], keys [t_k,b,n]); same
    parameters as the block it replaces (linear_q, linear_k, linear_att, normalize_scalar, normalize_bias)."""

    def __init__(self, att):
        super().__init__()
        self.num_units = att.num_units
        self.linear_q = _swap_leaf(att.linear_q)
        self.linear_k = _swap_leaf(att.linear_k)
        self.linear_att = att.linear_att
        self.normalize_scalar = att.normalize_scalar
        self.normalize_bias = att.normalize_bias
        self.register_buffer('mask', None)
        self._ctx_len = None

    @staticmethod
    def supports(m):
        return (type(m).__name__ == "BahdanauAttention" and getattr(m, "normalize", False)
                and not getattr(m, "batch_first", True) and hasattr(m, "linear_att")
                and getattr(getattr(m, "dropout", None), "p", 0) == 0)

    def set_mask(self, context_len, context):
        self._ctx_len = context_len.to(device=context.device, dtype=torch.int64).contiguous()
        self.mask = torch.arange(context.size(0), device=context.device).unsqueeze(0) >= self._ctx_len.unsqueeze(1)

    def forward(self, query, keys):
        if query.dim() != 3:
            raise NotImplementedError("single-step queries are an inference path")
        pq = self.linear_q(query.transpose(0, 1))          # [b, t_q, n]
        pk = self.linear_k(keys.transpose(0, 1))           # [b, t_k, n]
        a = self.linear_att.float()
        v = a / a.norm() * self.normalize_scalar.float()   # tiny [n] vector: autograd carries its chain rule
        context, probs = _AttnFn.apply(pq, pk, keys, v, self.normalize_bias, self._ctx_len)
        return context, probs.transpose(0, 1)

# --------------------------------------------------------------------------- #
# criteria
# --------------------------------------------------------------------------- #
class _SoftmaxCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, smoothing, padding_idx, scale):
        lg = logits if logits.is_contiguous() else logits.contiguous()
        loss, lse, _ = pf.softmax_ce_fwd(lg, target, smoothing, padding_idx, scale)
        ctx.saved = (lg, target, lse)
        ctx.cfg = (smoothing, padding_idx, scale)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        lg, target, lse = ctx.saved
        smoothing, padding_idx, scale = ctx.cfg
        up = dloss if dloss.dtype == torch.float32 else dloss.float()
        return pf.softmax_ce_bwd(lg, target, lse, smoothing, padding_idx, up.contiguous(), scale), None, None, None, None


class NativeCrossEntropyLoss(nn.Module):
    """torch.nn.CrossEntropyLoss() with mean reduction over [B, C] logits."""

    @staticmethod
    def supports(m):
        return (isinstance(m, nn.CrossEntropyLoss) and m.weight is None and m.reduction == "mean"
                and m.ignore_index == -100 and getattr(m, "label_smoothing", 0.0) == 0.0)

    def forward(self, logits, target):
        return _SoftmaxCEFn.apply(logits, target, 0.0, -1, 1.0 / logits.shape[0])


class NativeLabelSmoothing(nn.Module):
    """Label-smoothed NLL over [T, B, V] logits, PAD rows masked, sum divided by B
    (runtime/translation/seq2seq/train/smoothing.py:7-34)."""

    def __init__(self, padding_idx, smoothing):
        super().__init__()
        self.padding_idx = padding_idx
        self.smoothing = smoothing
        self.confidence = 1.0 - smoothing

    def forward(self, output, target):
        x = output.reshape(output.size(0) * output.size(1), -1)
        return _SoftmaxCEFn.apply(x, target, float(self.smoothing), int(self.padding_idx), 1.0 / output.size(1))


# --------------------------------------------------------------------------- #
# stage rewriting
# --------------------------------------------------------------------------- #
_LAYOUT_AWARE = (NativeConv2d, NativeReLU, NativeMaxPool2d, FusedAway, NativeBatchNorm2d, NativeConvGeneric,
                 NativeMaxPool3s2, NativeGlobalAvgPool)
_NATIVE_TYPES = _LAYOUT_AWARE + (NativeLinear, NativeDropout, NativeCrossEntropyLoss, NativeLabelSmoothing,
                                 NativeLSTM, NativeEmuBidirLSTM, NativeEmbedding, NativeBahdanauAttention,
                                 NativeBatchNorm2d, NativeConvGeneric, NativeMaxPool3s2, NativeGlobalAvgPool,
                                 NativeLayerNorm, NativeGELU, NativeCausalAttentionCore)


_PADDED_PRODUCERS = (NativeConv2d, NativeReLU, NativeMaxPool2d, NativeBatchNorm2d, NativeMaxPool3s2, NativeConvGeneric)
_PADDED_CONSUMERS = (NativeConv2d, NativeReLU, NativeMaxPool2d, NativeBatchNorm2d, NativeConvGeneric, NativeMaxPool3s2,
                     NativeGlobalAvgPool)


def _swap_leaf(m):
    if isinstance(m, _LAYOUT_AWARE + (NativeLinear, NativeDropout, NativeCrossEntropyLoss, NativeLabelSmoothing,
                                      NativeLSTM, NativeEmuBidirLSTM, NativeEmbedding, NativeBahdanauAttention,
                                      NativeCausalAttentionCore)):
        return m
    if NativeConv2d.supports(m):
        return NativeConv2d(m)
    if NativeConvGeneric.supports(m):
        return NativeConvGeneric(m)
    if NativeBatchNorm2d.supports(m):
        return NativeBatchNorm2d(m)
    if NativeMaxPool3s2.supports(m):
        return NativeMaxPool3s2()
    if NativeGlobalAvgPool.supports(m):
        return NativeGlobalAvgPool(m.kernel_size)
    if isinstance(m, nn.ReLU):
        return NativeReLU()
    if NativeMaxPool2d.supports(m):
        return NativeMaxPool2d()
    if NativeLinear.supports(m):
        return NativeLinear(m)
    if NativeLayerNorm.supports(m):
        return NativeLayerNorm(m)
    if isinstance(m, nn.GELU):
        return NativeGELU(m.approximate)
    if NativeCausalAttentionCore.supports(m):
        return NativeCausalAttentionCore(m)
    if NativeLSTM.supports(m):
        return NativeLSTM(m)
    if NativeEmuBidirLSTM.supports(m):
        return NativeEmuBidirLSTM(m)
    if NativeEmbedding.supports(m):
        return NativeEmbedding(m)
    if NativeBahdanauAttention.supports(m):
        return NativeBahdanauAttention(m)
    if isinstance(m, nn.Dropout):
        return NativeDropout(m.p)
    if NativeCrossEntropyLoss.supports(m):
        return NativeCrossEntropyLoss()
    if type(m).__name__ == "LabelSmoothing" and hasattr(m, "padding_idx") and hasattr(m, "smoothing"):
        return NativeLabelSmoothing(m.padding_idx, m.smoothing)
    return m


def _is_add(node):
    import operator
    if node.op == "call_function":
        return node.target in (operator.add, operator.iadd, torch.add)
    return node.op == "call_method" and node.target in ("add", "add_", "__add__", "__iadd__")


def _fuse_residual_tails(module, graph, mods):
    """BatchNorm -> add(shortcut) -> ReLU becomes one call of the BatchNorm module with the shortcut as its
    second argument; a value with two layout-aware consumers goes through a NativeFork.  Returns True when
    the graph was changed (the stage then has to run from the rewritten graph, not from its own forward)."""
    import operator
    changed = False

    def target_mod(node):
        return mods.get(node.target) if node.op == "call_module" else None

    def call_sites(target):
        return sum(1 for n in graph.nodes if n.op == "call_module" and n.target == target)

    for node in list(graph.nodes):
        if not _is_add(node) or node.kwargs or len(node.args) != 2 or len(node.users) != 1:
            continue
        a, b = node.args
        if not (hasattr(a, "op") and hasattr(b, "op")):
            continue
        relu = next(iter(node.users))
        if not isinstance(target_mod(relu), NativeReLU) or relu.args != (node,) or call_sites(relu.target) != 1:
            continue
        for bn_node, other in ((a, b), (b, a)):
            bm = target_mod(bn_node)
            if (isinstance(bm, NativeBatchNorm2d) and not bm.fuse_relu and len(bn_node.users) == 1
                    and len(bn_node.args) == 1 and call_sites(bn_node.target) == 1):
                with graph.inserting_before(relu):
                    fused = graph.call_module(bn_node.target, (bn_node.args[0], other))
                relu.replace_all_uses_with(fused)
                graph.erase_node(relu)
                graph.erase_node(node)
                graph.erase_node(bn_node)
                bm.fuse_relu = True
                changed = True
                break
    if not changed:
        return False
    k = 0
    for node in list(graph.nodes):
        if node.op not in ("placeholder", "call_module") or len(node.users) != 2:
            continue
        users = list(node.users)
        if not all(isinstance(target_mod(u), _PADDED_CONSUMERS) for u in users):
            continue
        name = "pd_fork%d" % k
        k += 1
        module.add_module(name, NativeFork())
        mods[name] = getattr(module, name)
        with graph.inserting_after(node):
            f = graph.call_module(name, (node,))
        with graph.inserting_after(f):
            g0 = graph.call_function(operator.getitem, (f, 0))
        with graph.inserting_after(g0):
            g1 = graph.call_function(operator.getitem, (f, 1))
        users[0].replace_input_with(node, g0)
        users[1].replace_input_with(node, g1)
    graph.lint()
    return True


def nativize(module):
    """Swap the leaf modules of a stage for native ones and plan fusions.

    The stage's own forward() keeps running as written, with one exception: a container in which a
    BatchNorm -> add -> ReLU tail (residual block) is found is replaced by a torch.fx GraphModule of its
    own trace, with that tail fused (parameter and buffer names are unchanged).  Otherwise the torch.fx
    trace is used only to prove that a fusion / layout choice is safe: a ReLU is folded into the producing
    conv, linear or batch norm when it is that node's only consumer, and a 4-D result stays in padded NHWC
    only when every consumer is layout aware.  Without a trace every native module emits plain contiguous
    tensors.
    """
    single = _swap_leaf(module)
    if single is not module:
        return single
    for n, child in list(module.named_children()):
        new = _swap_leaf(child)
        if new is child and not isinstance(child, _NATIVE_TYPES) and any(True for _ in child.children()):
            new = nativize(child)       # a container (residual block, attention block): plan it on its own
        if new is not child:
            setattr(module, n, new)
    try:
        import torch.fx as fx

        class _Tracer(fx.Tracer):
            def is_leaf_module(self, m, qualname):
                return True
        graph = _Tracer().trace(module)
    except Exception:
        return module
    mods = dict(module.named_modules())

    def target_mod(node):
        return mods.get(node.target) if node.op == "call_module" else None

    # 1. fold ReLU into its producer
    for node in graph.nodes:
        m = target_mod(node)
        if isinstance(m, (NativeConv2d, NativeLinear, NativeBatchNorm2d)) and len(node.users) == 1:
            user = next(iter(node.users))
            um = target_mod(user)
            if isinstance(um, NativeReLU) and user.args == (node,):
                # the same ReLU module instance must not be shared with another call site
                calls = [n for n in graph.nodes if n.op == "call_module" and n.target == user.target]
                if len(calls) == 1:
                    m.fuse_relu = True
                    parent, _, attr = user.target.rpartition(".")
                    setattr(mods[parent] if parent else module, attr, FusedAway())
                    mods[user.target] = FusedAway()
    # 1b. residual tails (BatchNorm -> add -> ReLU) and forks: these rewrite the graph
    result = module
    try:
        rewritten = _fuse_residual_tails(module, graph, mods)
    except Exception:
        rewritten = False
        graph = _Tracer().trace(module)
    if rewritten:
        result = fx.GraphModule(module, graph)
        result.train(module.training)
        # children in the order of the original module, so that parameters() / state_dict() keep their order
        kids = result._modules
        order = [k for k in module._modules if k in kids] + [k for k in kids if k not in module._modules]
        result._modules = type(kids)((k, kids[k]) for k in order)
    # 2. keep 4-D results in padded NHWC when every consumer (of every call site) understands it.  A nested
    # container that was planned before counts as a producer through the module that feeds its output,
    # and as a consumer when everything that reads its input is layout aware.
    import operator

    def producer_of(m):
        if isinstance(m, _PADDED_PRODUCERS):
            return m
        return getattr(m, "_pd_out_module", None) if m is not None else None

    def all_users_accept(node):
        frontier, ok = list(node.users), len(node.users) > 0
        while frontier and ok:
            u = frontier.pop()
            um = target_mod(u)
            if isinstance(um, (FusedAway, NativeFork)) or (u.op == "call_function" and u.target is operator.getitem):
                frontier.extend(u.users)
                ok = len(u.users) > 0
            elif not (isinstance(um, _PADDED_CONSUMERS) or getattr(um, "_pd_accepts_padded", False)):
                ok = False
        return ok

    decided = {}
    for node in graph.nodes:
        m = producer_of(target_mod(node))
        if m is None:
            continue
        decided[id(m)] = decided.get(id(m), True) and all_users_accept(node)
        m.out_nchw = not decided[id(m)]
    # what the enclosing container may assume about this one
    placeholders = [n for n in graph.nodes if n.op == "placeholder"]
    outputs = [n for n in graph.nodes if n.op == "output"]
    result._pd_accepts_padded = len(placeholders) == 1 and all_users_accept(placeholders[0])
    object.__setattr__(result, "_pd_out_module", None)     # plain attribute: not a registered submodule
    if len(outputs) == 1 and len(outputs[0].args) == 1 and hasattr(outputs[0].args[0], "op"):
        last = outputs[0].args[0]
        while isinstance(target_mod(last), FusedAway) and len(last.args) == 1 and len(last.users) == 1:
            last = last.args[0]
        m = producer_of(target_mod(last))
        if m is not None and len(last.users) == 1 and sum(1 for n in graph.nodes if n.op == "call_module"
                                                          and n.target == last.target) == 1:
            object.__setattr__(result, "_pd_out_module", m)
    return result
