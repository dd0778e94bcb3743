"""GPU parity of the contraction kernel at the layer shapes of VGG-16 (vgg16/gpus=8/stage0.py:10-31,
stage1.py:12-16), one case per distinct (H, Cin, Cout), all three passes, against torch fp32 - and of the
CTA-pair tiling against the single-CTA tiling on the shapes that qualify for pairs.

Small kernel tests never wrap the persistent tile loop past the SM count, never run the shared-memory ring across
tile boundaries at full depth and never reach the 224 x 224 tap-sharing path; these do.  Tolerance: bf16 results
within 2e-2 of the fp32 reference relative to the output scale; the two tilings within 1e-3 of each other.
"""
import ctypes

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from pipedream_b200 import functional as pf  # noqa: E402
from pipedream_b200 import _lib  # noqa: E402

DEV = "cuda"
torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_tf32 = False
TOL = 2e-2

# (batch, Cin, Cout, H): every distinct convolution of VGG-16 but the first (Cin = 3 runs as a patch matrix).
# Batches are the smallest that keep the wide layers on the CTA-pair path (at least 74 tiles of 256 x 256).
VGG_LAYERS = [(8, 64, 64, 224), (8, 64, 128, 112), (8, 128, 128, 112), (8, 128, 256, 56), (8, 256, 256, 56),
              (16, 256, 512, 28), (16, 512, 512, 28), (64, 512, 512, 14)]


def rnd(*shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(DEV).to(torch.bfloat16)


def rel_err(got, ref):
    return ((got.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-6)).item()


def pad_ref(x):
    return F.pad(x, (1, 1, 1, 1)).permute(0, 2, 3, 1).contiguous()


def set_pair_mode(mode):
    _lib.call("pd_gemm_set_pair_mode", ctypes.c_int(mode))


def run_layer(N, Cin, Cout, H):
    x = rnd(N, Cin, H, H, seed=1)
    w = rnd(Cout, Cin, 3, 3, seed=2, scale=(2.0 / (9 * Cin)) ** 0.5)
    wcl = w.permute(0, 2, 3, 1).contiguous()
    bias = rnd(Cout, seed=3)
    dy = rnd(N, Cout, H, H, seed=4)
    xp, dyp = pf.pack_pnhwc(x), pf.pack_pnhwc(dy)
    y = pf.conv2d_fwd(xp, wcl, 9 * Cin, Cout, bias, True)
    dx = pf.conv2d_dgrad(dyp, wcl, 9 * Cin, Cin, relu_aux=xp)
    dw = torch.empty(Cout, 9 * Cin, device=DEV, dtype=torch.float32)
    pf.conv2d_wgrad(xp, dyp, dw, 9 * Cin, accumulate=False)
    torch.cuda.synchronize()
    assert pf.gemm_poll_error() == 0, "a tcgen05 kernel reported a wait that ran out"
    return (x, w, bias, dy), (y, dx, dw)


@pytest.mark.parametrize("N,Cin,Cout,H", VGG_LAYERS)
def test_vgg_layer_shape(N, Cin, Cout, H):
    set_pair_mode(1)
    (x, w, bias, dy), (y, dx, dw) = run_layer(N, Cin, Cout, H)
    x32 = x.float().requires_grad_(True)
    w32 = w.float().requires_grad_(True)
    ref = F.conv2d(x32, w32, bias.float(), padding=1)
    pre = ref.detach()
    ref.backward(dy.float())
    e_y = rel_err(y, pad_ref(F.relu(pre)))
    e_dx = rel_err(dx, pad_ref(x32.grad * (x32.detach() > 0)))
    e_dw = rel_err(dw, w32.grad.permute(0, 2, 3, 1).reshape(Cout, 9 * Cin))
    assert torch.isfinite(y.float()).all() and torch.isfinite(dx.float()).all() and torch.isfinite(dw).all()
    assert e_y <= TOL and e_dx <= TOL and e_dw <= TOL, (e_y, e_dx, e_dw)
    # the padding ring stays zero
    assert (y[:, 0] == 0).all() and (y[:, -1] == 0).all() and (y[:, :, 0] == 0).all() and (y[:, :, -1] == 0).all()


@pytest.mark.parametrize("N,Cin,Cout,H", [s for s in VGG_LAYERS if s[1] >= 256 or s[2] >= 256])
def test_pair_tiling_matches_single(N, Cin, Cout, H):
    try:
        set_pair_mode(1)
        _, (y2, dx2, dw2) = run_layer(N, Cin, Cout, H)
        set_pair_mode(0)
        _, (y1, dx1, dw1) = run_layer(N, Cin, Cout, H)
    finally:
        set_pair_mode(1)
    assert rel_err(y2, y1) <= 1e-3, rel_err(y2, y1)
    assert rel_err(dx2, dx1) <= 1e-3, rel_err(dx2, dx1)
    assert rel_err(dw2, dw1) <= 1e-3, rel_err(dw2, dw1)      # split-K counts differ: fp32 atomics in another order


@pytest.mark.parametrize("M,N,K", [(19000, 512, 200), (25000, 256, 64), (40000, 768, 136)])
def test_pair_gemm_ragged(M, N, K):
    """Plain GEMMs on the pair path with M not a multiple of 256 and a K tail."""
    set_pair_mode(1)
    a = rnd(M, K, seed=5)
    b = rnd(N, K, seed=6)
    bias = rnd(N, seed=7)
    out = pf.gemm_nt(a, b, bias=bias, relu=True)
    ref = F.relu(a.float() @ b.float().t() + bias.float())
    assert rel_err(out, ref) <= TOL, rel_err(out, ref)
    bt = b.t().contiguous()                      # [K, N]
    out = pf.gemm_nn(a, bt)
    assert rel_err(out, a.float() @ bt.float()) <= TOL
    # weight-gradient form: out[M2, N] = a2[K2, M2]^T . b2[K2, N], wide in both directions
    a2 = rnd(M, 512, seed=8)
    b2 = rnd(M, N, seed=9)
    dw = torch.empty(512, N, device=DEV)
    pf.gemm_tn(a2, b2, dw, accumulate=False)
    assert rel_err(dw, a2.float().t() @ b2.float()) <= TOL
    assert pf.gemm_poll_error() == 0
