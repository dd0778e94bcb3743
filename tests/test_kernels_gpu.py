"""GPU parity tests of the individual C-ABI kernels against torch fp32 references.

Tolerances: fp32 kernels 1e-4 relative to the output scale (summation order
differs); bf16 kernels 2e-2 (the bar for bf16 results).
"""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from pipedream_b200 import functional as pf  # noqa: E402

DEV = "cuda"
# the fp32 references must be real fp32, not TF32
torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_tf32 = False
TOL = {torch.float32: 2e-4, torch.bfloat16: 2e-2}


def rel_err(got, ref):
    got = got.float()
    ref = ref.float()
    return ((got - ref).abs().max() / ref.abs().max().clamp_min(1e-6)).item()


def check(got, ref, dtype, what):
    assert got.shape == ref.shape, "%s: shape %s vs %s" % (what, tuple(got.shape), tuple(ref.shape))
    assert torch.isfinite(got.float()).all(), "%s: non-finite values" % what
    e = rel_err(got, ref)
    assert e <= TOL[dtype], "%s: relative error %.3e > %.1e" % (what, e, TOL[dtype])
    assert pf.gemm_poll_error() == 0, "%s: tcgen05 kernel reported a wait that ran out" % what


def rnd(*shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(DEV).to(dtype)


def pad_ref(x):
    """torch reference of the padded-NHWC layout."""
    return F.pad(x, (1, 1, 1, 1)).permute(0, 2, 3, 1).contiguous()


# ------------------------------------------------------------------ layout
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", [(2, 3, 8, 8), (3, 64, 14, 14), (1, 40, 5, 37)])
def test_pack_unpack(dtype, shape):
    x = rnd(*shape, dtype=dtype, seed=1)
    pad = pf.pack_pnhwc(x)
    assert torch.equal(pad, pad_ref(x))
    assert torch.equal(pf.unpack_pnhwc(pad), x)
    view = pf.nchw_view(pad, *shape)
    assert torch.equal(view, x)
    assert pf.padded_of(view).data_ptr() == pad.data_ptr()
    # channels-last source and dtype conversion
    xcl = x.float().contiguous(memory_format=torch.channels_last)
    pad2 = pf.pack_pnhwc(xcl, dtype=torch.bfloat16)
    assert torch.equal(pad2, pad_ref(x.float()).to(torch.bfloat16))


def test_im2col():
    x = rnd(2, 3, 9, 11, dtype=torch.float32, seed=2)
    col = pf.im2col3x3(x, 32, torch.float32)
    N, C, H, W = x.shape
    ref = F.unfold(x, 3, padding=1).view(N, C, 9, H, W).permute(0, 3, 4, 2, 1).reshape(N, H, W, 27)
    full = torch.zeros(N, H + 2, W + 2, 32, device=DEV)
    full[:, 1:-1, 1:-1, :27] = ref
    assert torch.equal(col.view(N, H + 2, W + 2, 32), full)


@pytest.mark.parametrize("layout", ["nchw", "channels_last"])
def test_im2col_three_channels_bf16(layout):
    """The first layer's patch matrix as the training path builds it: fp32 images, bf16 rows of 32."""
    x = rnd(3, 3, 10, 14, dtype=torch.float32, seed=21)
    if layout == "channels_last":
        x = x.contiguous(memory_format=torch.channels_last)
    col = pf.im2col3x3(x, 32, torch.bfloat16)
    N, C, H, W = x.shape
    ref = F.unfold(x.contiguous(), 3, padding=1).view(N, C, 9, H, W).permute(0, 3, 4, 2, 1).reshape(N, H, W, 27)
    full = torch.zeros(N, H + 2, W + 2, 32, device=DEV)
    full[:, 1:-1, 1:-1, :27] = ref
    assert torch.equal(col.view(N, H + 2, W + 2, 32), full.to(torch.bfloat16))


# ------------------------------------------------------------------ pointwise
@pytest.mark.parametrize("C,H,W", [(64, 12, 16), (128, 6, 10), (512, 4, 4), (8, 2, 2)])
def test_maxpool_bwd_with_bias_colsum(C, H, W):
    """Pool backward that also reduces the bias gradient of the conv+ReLU in front of it."""
    dtype = torch.bfloat16
    xr = F.relu(rnd(3, C, H, W, dtype=dtype, seed=31))
    xrp = pf.pack_pnhwc(xr)
    assert pf.maxpool2_bwd_colsum_ok(xrp)
    g = rnd(3, C, H // 2, W // 2, dtype=dtype, seed=32)
    xr32 = xr.float().requires_grad_(True)
    F.max_pool2d(xr32, 2).backward(g.float())
    want = (xr32.grad * (xr32 > 0)).to(dtype)
    dx, partial = pf.maxpool2_bwd_colsum(xrp, pf.pack_pnhwc(g), True)
    assert torch.equal(dx, pad_ref(want))
    assert torch.equal(dx, pf.maxpool2_bwd(xrp, pf.pack_pnhwc(g), False, True))
    cs = torch.full((C,), 2.0, device=DEV)
    pf.colsum_finish(partial, cs, True)
    check(cs, want.float().sum((0, 2, 3)) + 2.0, torch.float32, "colsum accumulate")
    pf.colsum_finish(partial, cs, False)
    check(cs, want.float().sum((0, 2, 3)), torch.float32, "colsum")
    assert not pf.maxpool2_bwd_colsum_ok(pf.pack_pnhwc(rnd(1, 24, 4, 4, dtype=dtype, seed=33)))   # 256 % 3 != 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_relu_pool(dtype):
    x = rnd(2, 64, 12, 16, dtype=dtype, seed=3)
    xp = pf.pack_pnhwc(x)
    y = pf.relu(xp)
    assert torch.equal(y, pad_ref(F.relu(x)))
    dy = rnd(2, 14, 18, 64, dtype=dtype, seed=4)
    assert torch.equal(pf.relu_bwd(dy, y), dy * (y > 0))
    # max-pool forward, both output layouts
    xr = F.relu(x)
    xrp = pf.pack_pnhwc(xr)
    ref = F.max_pool2d(xr.float(), 2).to(dtype)
    assert torch.equal(pf.maxpool2_fwd(xrp, True), ref)
    assert torch.equal(pf.maxpool2_fwd(xrp, False), pad_ref(ref))
    # backward against autograd (ties between zeros go to the first element on both sides)
    xr32 = xr.float().requires_grad_(True)
    g = rnd(2, 64, 6, 8, dtype=dtype, seed=5)
    F.max_pool2d(xr32, 2).backward(g.float())
    got = pf.maxpool2_bwd(xrp, g.contiguous(), True, False)
    assert torch.equal(got, pad_ref(xr32.grad.to(dtype)))
    got2 = pf.maxpool2_bwd(xrp, pf.pack_pnhwc(g), False, True)
    assert torch.equal(got2, pad_ref((xr32.grad * (xr32 > 0)).to(dtype)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("C", [64, 96, 512, 1000, 3072, 4104])
def test_relu_bwd_colsum(dtype, C):
    rows = 777
    dy = rnd(rows, C, dtype=dtype, seed=6)
    y = rnd(rows, C, dtype=dtype, seed=7)
    dx = torch.empty_like(dy)
    cs = torch.zeros(C, device=DEV)
    pf.relu_bwd_colsum(dy, y, dx, cs, False)
    ref = dy * (y > 0)
    assert torch.equal(dx, ref)
    check(cs, ref.float().sum(0), torch.float32, "colsum")
    pf.relu_bwd_colsum(dy, None, None, cs, True)
    check(cs, ref.float().sum(0) + dy.float().sum(0), torch.float32, "colsum accumulate")


def test_dropout():
    x = torch.ones(1 << 20, device=DEV)
    y, m = pf.dropout_fwd(x, 0.5, 1234, 0)
    keep = m.float().mean().item()
    assert abs(keep - 0.5) < 5e-3
    assert torch.equal(y, m.float() * 2.0)
    y2, m2 = pf.dropout_fwd(x, 0.5, 1234, 1 << 20)
    assert not torch.equal(m, m2)
    assert torch.equal(pf.dropout_bwd(x, m, 0.5), y)
    y0, m0 = pf.dropout_fwd(x, 0.0, 1, 0)
    assert torch.equal(y0, x)


# ------------------------------------------------------------------ criteria
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_cross_entropy(dtype):
    B, C = 64, 1000
    logits = (rnd(B, C, dtype=dtype, seed=8) * 3).contiguous()
    target = torch.randint(0, C, (B,), generator=torch.Generator().manual_seed(9)).to(DEV)
    loss, lse, _ = pf.softmax_ce_fwd(logits, target, 0.0, -1, 1.0 / B)
    l32 = logits.float().requires_grad_(True)
    ref = F.cross_entropy(l32, target)
    ref.backward()
    assert abs(loss.item() - ref.item()) <= 1e-5 * abs(ref.item()) + 1e-6
    d = pf.softmax_ce_bwd(logits, target, lse, 0.0, -1, None, 1.0 / B)
    check(d, l32.grad, dtype, "ce grad")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_label_smoothing(dtype):
    T, B, C = 7, 16, 32320
    logits = rnd(T * B, C, dtype=dtype, seed=10)
    target = torch.randint(0, C, (T * B,), generator=torch.Generator().manual_seed(11)).to(DEV)
    target[::5] = 0   # padding
    sm = 0.1
    loss, lse, _ = pf.softmax_ce_fwd(logits, target, sm, 0, 1.0 / B)
    l32 = logits.float().requires_grad_(True)
    logp = F.log_softmax(l32, dim=-1)
    mask = target != 0
    nll = -logp.gather(1, target.unsqueeze(1)).squeeze(1)[mask]
    smooth = -logp.mean(-1)[mask]
    ref = ((1 - sm) * nll + sm * smooth).sum() / B
    ref.backward()
    assert abs(loss.item() - ref.item()) <= 2e-5 * abs(ref.item())
    up = torch.tensor(2.0, device=DEV)
    d = pf.softmax_ce_bwd(logits, target, lse, sm, 0, up, 1.0 / B)
    check(d, 2 * l32.grad, dtype, "label smoothing grad")


# ------------------------------------------------------------------ sequence
def test_revert_varlen_and_mask():
    T, B, Fd = 9, 5, 24
    x = rnd(T, B, Fd, dtype=torch.bfloat16, seed=12)
    lengths = torch.tensor([9, 7, 4, 2, 1], dtype=torch.int64)
    ref = torch.zeros_like(x)
    for b in range(B):
        L = int(lengths[b])
        ref[:L, b] = x[:L, b].flip(0)
    got = pf.revert_varlen(x, lengths.to(DEV))
    assert torch.equal(got, ref)
    m = pf.length_mask(lengths.to(DEV), T, torch.uint8)
    refm = (torch.arange(T).unsqueeze(1) < lengths.unsqueeze(0)).to(torch.uint8)
    assert torch.equal(m.cpu(), refm)
    x3 = rnd(T, B, 3, dtype=torch.float32, seed=13)   # 12-byte rows: scalar path
    ref3 = torch.zeros_like(x3)
    for b in range(B):
        L = int(lengths[b])
        ref3[:L, b] = x3[:L, b].flip(0)
    assert torch.equal(pf.revert_varlen(x3, lengths.to(DEV)), ref3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_embedding(dtype):
    V, D = 1000, 64
    table = rnd(V, D, dtype=dtype, seed=14)
    ids = torch.randint(0, V, (6, 7), generator=torch.Generator().manual_seed(15)).to(DEV)
    ids[0, :3] = 0
    assert torch.equal(pf.embedding_fwd(ids, table), table[ids])
    dy = rnd(6, 7, D, dtype=dtype, seed=16)
    dt_ = torch.zeros(V, D, device=DEV)
    pf.embedding_bwd(ids, dy, dt_, 0)
    ref = torch.zeros(V, D, device=DEV)
    ref.index_add_(0, ids.view(-1), dy.float().view(-1, D))
    ref[0] = 0
    check(dt_, ref, torch.float32, "embedding grad")


# ------------------------------------------------------------------ contractions
GEMM_SHAPES = [(256, 256, 128), (128, 64, 64), (64, 1000, 4096), (300, 200, 32), (130, 520, 1000)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_nt(dtype, M, N, K):
    a = rnd(M, K, dtype=dtype, seed=20)
    b = rnd(N, K, dtype=dtype, seed=21)
    bias = rnd(N, dtype=dtype, seed=22)
    ref = a.float() @ b.float().t()
    check(pf.gemm_nt(a, b), ref, dtype, "gemm_nt")
    check(pf.gemm_nt(a, b, bias=bias, relu=True), F.relu(ref + bias.float()), dtype, "gemm_nt bias relu")


@pytest.mark.parametrize("M,N,K", [(64, 4096, 25088), (64, 1000, 4096), (33, 520, 4160), (128, 4096, 4096)])
def test_gemm_nt_short_and_wide_splits_k(M, N, K):
    """Linear layers at a small batch take the split-K path (fp32 partial sums in a workspace, bias / ReLU / bf16
    conversion in a second kernel); with the deterministic switch they take the plain one."""
    dtype = torch.bfloat16
    a = rnd(M, K, dtype=dtype, seed=40) * 0.1
    b = rnd(N, K, dtype=dtype, seed=41) * 0.1
    bias = rnd(N, dtype=dtype, seed=42)
    ref = a.float() @ b.float().t()
    got = pf.gemm_nt(a, b, bias=bias, relu=True)
    check(got, F.relu(ref + bias.float()), dtype, "gemm_nt split-K bias relu")
    check(pf.gemm_nt(a, b, out_dtype=torch.float32), ref, dtype, "gemm_nt split-K fp32 out")
    prev = pf.set_deterministic(True)
    try:
        plain = pf.gemm_nt(a, b, bias=bias, relu=True)
        again = pf.gemm_nt(a, b, bias=bias, relu=True)
    finally:
        pf.set_deterministic(prev)
    assert torch.equal(plain, again)
    check(plain, F.relu(ref + bias.float()), dtype, "gemm_nt plain")
    assert pf.gemm_poll_error() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_nn(dtype, M, N, K):
    a = rnd(M, K, dtype=dtype, seed=23)
    b = rnd(K, N, dtype=dtype, seed=24)
    ref = a.float() @ b.float()
    check(pf.gemm_nn(a, b), ref, dtype, "gemm_nn")
    aux = rnd(M, N, dtype=dtype, seed=25)
    check(pf.gemm_nn(a, b, relu_aux=aux), ref * (aux > 0), dtype, "gemm_nn masked")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (128, 64, 64), (1000, 4096, 64), (304, 200, 32), (136, 520, 1000),
                                   (64, 64, 5000)])
def test_gemm_tn(dtype, M, N, K):
    a = rnd(K, M, dtype=dtype, seed=26)
    b = rnd(K, N, dtype=dtype, seed=27)
    ref = a.float().t() @ b.float()
    out = torch.full((M, N), 7.0, device=DEV)
    check(pf.gemm_tn(a, b, out, accumulate=False, split_k=1), ref, dtype, "gemm_tn")
    out = torch.full((M, N), 7.0, device=DEV)
    check(pf.gemm_tn(a, b, out, accumulate=False), ref, dtype, "gemm_tn auto split")
    check(pf.gemm_tn(a, b, out, accumulate=True, split_k=3), 2 * ref, dtype, "gemm_tn accumulate")


CONV_SHAPES = [(2, 64, 128, 16, 16), (3, 128, 64, 14, 14), (1, 64, 64, 7, 9), (2, 256, 512, 8, 8)]


def conv_weight(cout, cin, dtype, seed):
    w = rnd(cout, cin, 3, 3, dtype=dtype, seed=seed) * (2.0 / (9 * cin)) ** 0.5
    wcl = w.permute(0, 2, 3, 1).contiguous()   # [Cout][r][s][Cin]
    return w, wcl


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("N,Cin,Cout,H,W", CONV_SHAPES)
def test_conv_fwd(dtype, N, Cin, Cout, H, W):
    x = rnd(N, Cin, H, W, dtype=dtype, seed=30)
    w, wcl = conv_weight(Cout, Cin, dtype, 31)
    bias = rnd(Cout, dtype=dtype, seed=32)
    ref = F.conv2d(x.float(), w.float(), bias.float(), padding=1)
    xp = pf.pack_pnhwc(x)
    y = pf.conv2d_fwd(xp, wcl, 9 * Cin, Cout, bias, False)
    check(y, pad_ref(ref), dtype, "conv fwd")
    y = pf.conv2d_fwd(xp, wcl, 9 * Cin, Cout, bias, True)
    check(y, pad_ref(F.relu(ref)), dtype, "conv fwd relu")
    assert (y[:, 0] == 0).all() and (y[:, -1] == 0).all() and (y[:, :, 0] == 0).all() and (y[:, :, -1] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("N,Cin,Cout,H,W", CONV_SHAPES)
def test_conv_bwd(dtype, N, Cin, Cout, H, W):
    x = rnd(N, Cin, H, W, dtype=dtype, seed=33)
    w, wcl = conv_weight(Cout, Cin, dtype, 34)
    dy = rnd(N, Cout, H, W, dtype=dtype, seed=35)
    x32 = x.float().requires_grad_(True)
    w32 = w.float().requires_grad_(True)
    F.conv2d(x32, w32, None, padding=1).backward(dy.float())
    xp, dyp = pf.pack_pnhwc(x), pf.pack_pnhwc(dy)
    dx = pf.conv2d_dgrad(dyp, wcl, 9 * Cin, Cin)
    check(dx, pad_ref(x32.grad), dtype, "conv dgrad")
    dxm = pf.conv2d_dgrad(dyp, wcl, 9 * Cin, Cin, relu_aux=xp)
    check(dxm, pad_ref(x32.grad * (x32 > 0)), dtype, "conv dgrad masked")
    ref_dw = w32.grad.permute(0, 2, 3, 1).reshape(Cout, 9 * Cin)
    dw = torch.full((Cout, 9 * Cin), 3.0, device=DEV)
    check(pf.conv2d_wgrad(xp, dyp, dw, 9 * Cin, accumulate=False, split_k=1), ref_dw, dtype, "conv wgrad")
    dw = torch.full((Cout, 9 * Cin), 3.0, device=DEV)
    check(pf.conv2d_wgrad(xp, dyp, dw, 9 * Cin, accumulate=False), ref_dw, dtype, "conv wgrad auto split")
    check(pf.conv2d_wgrad(xp, dyp, dw, 9 * Cin, accumulate=True, split_k=2), 2 * ref_dw, dtype, "conv wgrad acc")


# ------------------------------------------------------------------ optimizer
def _call_sgd(arena, V, rs, ws, master, grad, mom, n, first, **kw):
    from pipedream_b200._lib import call
    import ctypes
    p = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
    call("pd_opt_sgd_multi_tensor", p(arena), arena.shape[1], rs, ws, pf.dt(arena), p(master), p(grad), p(mom), n,
         kw["lr"], kw["momentum"], kw.get("dampening", 0.0), kw["weight_decay"], int(kw.get("nesterov", False)),
         int(first), kw.get("grad_scale", 1.0), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("nesterov", [False, True])
def test_sgd_ring_fp32(nesterov):
    n, V = 1000 + 3, 3
    stride = 1008
    w0 = rnd(n, dtype=torch.float32, seed=40)
    arena = torch.zeros(V, stride, device=DEV)
    arena[0, :n] = w0
    mom = torch.zeros(stride, device=DEV)
    p_ref = torch.nn.Parameter(w0.cpu().clone())
    opt = torch.optim.SGD([p_ref], lr=0.05, momentum=0.9, weight_decay=5e-4, nesterov=nesterov)
    for step in range(4):
        g = rnd(n, dtype=torch.float32, seed=41 + step)
        p_ref.grad = g.cpu().clone()
        opt.step()
        gbuf = torch.zeros(stride, device=DEV)
        gbuf[:n] = g
        _call_sgd(arena, V, step % V, (step + 1) % V, None, gbuf, mom, n, step == 0, lr=0.05, momentum=0.9,
                  weight_decay=5e-4, nesterov=nesterov)
        got = arena[(step + 1) % V, :n].cpu()
        assert torch.allclose(got, p_ref.data, rtol=1e-6, atol=1e-7), "step %d" % step


def test_sgd_ring_bf16_master():
    n, V, stride = 4096, 2, 4096
    w0 = rnd(n, dtype=torch.float32, seed=50)
    master = w0.clone()
    arena = torch.zeros(V, stride, device=DEV, dtype=torch.bfloat16)
    arena[0] = w0.to(torch.bfloat16)
    mom = torch.zeros(stride, device=DEV)
    p_ref = torch.nn.Parameter(w0.cpu().clone())
    opt = torch.optim.SGD([p_ref], lr=0.01, momentum=0.9, weight_decay=1e-4)
    for step in range(3):
        g = rnd(n, dtype=torch.float32, seed=51 + step)
        p_ref.grad = g.cpu().clone()
        opt.step()
        _call_sgd(arena, V, step % V, (step + 1) % V, master, g.contiguous(), mom, n, step == 0, lr=0.01,
                  momentum=0.9, weight_decay=1e-4)
        assert torch.allclose(master.cpu(), p_ref.data, rtol=1e-6, atol=1e-7)
        assert torch.equal(arena[(step + 1) % V].cpu(), p_ref.data.to(torch.bfloat16)) or \
            rel_err(arena[(step + 1) % V].cpu(), p_ref.data) < 1e-2


def test_adam_ring():
    from pipedream_b200._lib import call
    import ctypes
    n, V, stride = 1000, 2, 1000
    w0 = rnd(n, dtype=torch.float32, seed=60)
    arena = torch.zeros(V, stride, device=DEV)
    arena[0] = w0
    m = torch.zeros(stride, device=DEV)
    v = torch.zeros(stride, device=DEV)
    p_ref = torch.nn.Parameter(w0.cpu().clone())
    opt = torch.optim.Adam([p_ref], lr=2e-3, betas=(0.9, 0.999), weight_decay=1e-4)
    p = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
    for step in range(5):
        g = rnd(n, dtype=torch.float32, seed=61 + step)
        p_ref.grad = g.cpu().clone()
        opt.step()
        call("pd_opt_adam_multi_tensor", p(arena), stride, step % V, (step + 1) % V, 0, None, p(g), p(m), p(v), n,
             2e-3, 0.9, 0.999, 1e-8, 1e-4, step + 1, 1.0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        got = arena[(step + 1) % V].cpu()
        assert torch.allclose(got, p_ref.data, rtol=2e-5, atol=1e-6), "step %d" % step


# ------------------------------------------------------------------ LSTM
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("T,B,I,H", [(5, 8, 64, 64), (12, 16, 128, 64), (1, 4, 64, 128), (7, 128, 256, 1024),
                                     (4, 100, 64, 320), (6, 32, 64, 256)])
def test_lstm_layer(dtype, T, B, I, H):
    """NativeLSTM forward and every gradient against torch.nn.LSTM (fp32 autograd on the same weights).  In bf16
    the forward recurrence of all but the T = 1 case runs as the whole-sequence cooperative kernel (8, 128 and 40
    CTAs; the (7, 128, 256, 1024) case is the translation model's layer shape and wraps the stage ring)."""
    from pipedream_b200 import layers
    torch.manual_seed(3)
    ref = torch.nn.LSTM(I, H).cuda()
    nat = torch.nn.LSTM(I, H).cuda().to(dtype)
    ref.load_state_dict({k: v.float() for k, v in nat.state_dict().items()})
    nat = layers.NativeLSTM(nat)
    x = rnd(T, B, I, dtype=dtype, seed=70)
    dy = rnd(T, B, H, dtype=dtype, seed=71)
    xr = x.float().detach().clone().requires_grad_(True)
    yr, _ = ref(xr)
    yr.backward(dy.float())
    xn = x.detach().clone().requires_grad_(True)
    yn, (hn, _) = nat(xn)
    yn.backward(dy)
    tol = TOL[dtype] if dtype == torch.bfloat16 else 1e-4
    check(yn, yr, dtype, "lstm y")
    assert torch.equal(hn[0], yn[-1])
    check(xn.grad, xr.grad, dtype, "lstm dx")
    for name in ("weight_ih_l0", "weight_hh_l0", "bias_ih_l0", "bias_hh_l0"):
        g, gr = getattr(nat, name)._pd_grad, getattr(ref, name).grad
        if T == 1 and name == "weight_hh_l0":
            assert float(g.abs().max()) == 0.0
            continue
        e = rel_err(g, gr)
        assert e <= 2 * tol, "%s: %.3e" % (name, e)


@pytest.mark.parametrize("T,B,H", [(9, 128, 1024), (6, 64, 256), (5, 96, 512)])
def test_lstm_halves_side_by_side_equal_one_launch(T, B, H):
    """The backward recurrence of a batch of 64..128 rows runs as two launches on two streams (rows b0 .. b0 + B/2 - 1
    of the same tensors): gate gradients equal to the single launch up to the order of the fp32 reductions.  The
    forward entry point for a row range is checked directly: two calls on the halves give the single launch's
    results bit for bit."""
    import ctypes
    from pipedream_b200 import _lib
    dtype = torch.bfloat16
    gx = rnd(T * B, 4 * H, dtype=dtype, seed=80) * 0.5
    w = rnd(4 * H, H, dtype=dtype, seed=81) * 0.05
    b = rnd(4 * H, dtype=dtype, seed=82) * 0.1
    dy = rnd(T, B, H, dtype=dtype, seed=83) * 0.1
    assert pf._lstm_halves(B, dtype) == ((0, B // 2), (B // 2, B // 2))
    y1, act1, c1 = pf.lstm_fwd(gx, w, b, T, B, H)
    dg2 = pf.lstm_bwd(dy, w, act1, c1)
    prev, pf._LSTM_SPLIT = pf._LSTM_SPLIT, False
    try:
        assert pf._lstm_halves(B, dtype) is None
        dg1 = pf.lstm_bwd(dy, w, act1, c1)
    finally:
        pf._LSTM_SPLIT = prev
    e = rel_err(dg2, dg1)
    print("two launches vs one, gate gradients: %.2e" % e)
    assert e <= 1e-2
    # forward on row ranges
    y2, act2, c2 = torch.empty_like(y1), torch.empty_like(act1), torch.empty_like(c1)
    ws = torch.zeros(128, dtype=torch.int32, device=DEV)
    p = lambda t: ctypes.c_void_p(t.data_ptr())          # noqa: E731
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for i, b0 in enumerate((0, B // 2)):
        assert _lib.call_or_decline("pd_lstm_fwd_rows", 1, p(gx), p(w), p(b), T, B, b0, B // 2, H, p(y2), p(act2), p(c2),
                                    ctypes.c_void_p(ws.data_ptr() + 256 * i), st)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2) and torch.equal(act1, act2) and torch.equal(c1, c2)
    assert pf.gemm_poll_error() == 0


def test_emu_bidir_lstm_and_embedding():
    """The swapped bidirectional encoder layer and embedding against their torch formulations."""
    from pipedream_b200 import layers, gnmt_blocks
    torch.manual_seed(4)
    T, B, H, V = 7, 6, 64, 50
    emb = torch.nn.Embedding(V, H, padding_idx=0).cuda()
    emu = gnmt_blocks.EmuBidirLSTM(H, H).cuda()
    lengths = torch.tensor([7, 6, 4, 4, 2, 1])
    ids = torch.randint(1, V, (T, B), generator=torch.Generator().manual_seed(5))
    for b in range(B):
        ids[lengths[b]:, b] = 0
    ids = ids.cuda()
    import copy
    nemb, nemu = layers.nativize(copy.deepcopy(emb)), layers.nativize(copy.deepcopy(emu))
    assert isinstance(nemb, layers.NativeEmbedding) and isinstance(nemu, layers.NativeEmuBidirLSTM)
    out_ref = gnmt_blocks.emu_bidir_reference(emu, emb(ids), lengths)
    out = nemu(nemb(ids), lengths.cuda())
    check(out, out_ref, torch.float32, "emu bidir")
    dy = rnd(T, B, 2 * H, dtype=torch.float32, seed=72)
    out_ref.backward(dy)
    out.backward(dy)
    check(nemb.weight._pd_grad, emb.weight.grad, torch.float32, "embedding grad")
    check(nemu.layer2.weight_hh_l0._pd_grad, emu.layer2.weight_hh_l0.grad, torch.float32, "reverse w_hh grad")
    check(nemu.layer1.weight_ih_l0._pd_grad, emu.layer1.weight_ih_l0.grad, torch.float32, "forward w_ih grad")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_bahdanau_attention(dtype):
    """Fused additive attention (forward, and every gradient) against the torch formulation of the block."""
    import copy
    from pipedream_b200 import layers, gnmt_blocks
    torch.manual_seed(6)
    tq, tk, b, n = 7, 9, 5, 64
    ref = gnmt_blocks.BahdanauAttention(n, n, n).cuda()
    with torch.no_grad():
        ref.normalize_bias.uniform_(-0.1, 0.1)
    nat = copy.deepcopy(ref).to(dtype)
    ref.load_state_dict({k: v.float() for k, v in nat.state_dict().items() if v is not None}, strict=False)
    nat = layers.nativize(nat)
    assert isinstance(nat, layers.NativeBahdanauAttention) and isinstance(nat.linear_q, layers.NativeLinear)
    q = rnd(tq, b, n, dtype=dtype, seed=80)
    k = rnd(tk, b, n, dtype=dtype, seed=81)
    lens = torch.tensor([9, 7, 4, 2, 1]).cuda()
    dctx = rnd(tq, b, n, dtype=dtype, seed=82)
    qr, kr = q.float().detach().clone().requires_grad_(True), k.float().detach().clone().requires_grad_(True)
    ref.set_mask(lens, kr)
    cr, pr = ref(qr, kr)
    cr.backward(dctx.float())
    qn, kn = q.detach().clone().requires_grad_(True), k.detach().clone().requires_grad_(True)
    nat.set_mask(lens, kn)
    cn, pn = nat(qn, kn)
    cn.backward(dctx)
    check(pn, pr, dtype, "attention probs")
    check(cn, cr, dtype, "attention context")
    check(qn.grad, qr.grad, dtype, "attention dquery")
    check(kn.grad, kr.grad, dtype, "attention dkeys")
    tol = 5e-2 if dtype == torch.bfloat16 else 1e-3
    for name in ("linear_att", "normalize_scalar", "normalize_bias"):
        e = rel_err(getattr(nat, name).grad, getattr(ref, name).grad)
        assert e <= tol, "%s: %.3e" % (name, e)
    for name in ("linear_q", "linear_k"):
        e = rel_err(getattr(nat, name).weight._pd_grad, getattr(ref, name).weight.grad)
        assert e <= tol, "%s: %.3e" % (name, e)


def test_no_memory_growth_across_steps():
    """Nothing saved for backward may keep a step alive after its backward ran (an output stored on the autograd
    context next to being returned forms a cycle through grad_fn that no collector sees)."""
    from pipedream_b200 import layers
    torch.manual_seed(0)
    lstm = layers.NativeLSTM(torch.nn.LSTM(64, 64).cuda().to(torch.bfloat16))
    lin = layers.NativeLinear(torch.nn.Linear(64, 64).cuda().to(torch.bfloat16))
    relu = layers.NativeReLU()
    base = None
    for i in range(8):
        x = rnd(12, 16, 64, dtype=torch.bfloat16, seed=80 + i).requires_grad_(True)
        y, _ = lstm(x)
        z = relu(lin(y).view(-1, 64))          # 2-D ReLU path
        z.float().sum().backward()
        del x, y, z
        torch.cuda.synchronize()
        if i == 3:
            base = torch.cuda.memory_allocated()
    assert torch.cuda.memory_allocated() <= base, (torch.cuda.memory_allocated(), base)
