"""Transformer pieces (LayerNorm, GELU) against torch, and a small GPT-style decoder through a two-stage
pipeline with double-buffered weights (2BW: two versions, one optimizer step per two minibatches) against the
CPU oracle of the same pipeline.  The reference has no transformer stages, so the oracle here is self-consistent
(same builder, plain torch modules, fp32) rather than pinned to reference outputs."""
import copy

import pytest
import torch
import torch.nn.functional as F

# whole-run comparisons: weight gradients without the run-to-run varying split (see conftest.py)
pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("deterministic_weight_gradients")]

from oracle import pipedream_oracle as oracle            # noqa: E402
from pipedream_b200 import layers, stages                # noqa: E402
from pipedream_b200 import functional as pf              # noqa: E402

torch.backends.cuda.matmul.allow_tf32 = False
TOL = {torch.float32: 2e-4, torch.bfloat16: 2e-2}


def rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-12)).item()


def rnd(*shape, seed):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)).cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("rows,C", [(37, 64), (1000, 1024), (5, 200)])
def test_layernorm(dtype, rows, C):
    ref = torch.nn.LayerNorm(C).cuda()
    with torch.no_grad():
        ref.weight.uniform_(0.5, 1.5)
        ref.bias.uniform_(-0.5, 0.5)
    nat = layers.NativeLayerNorm(copy.deepcopy(ref).to(dtype))
    ref.load_state_dict({k: v.float() for k, v in nat.state_dict().items()})
    x = (rnd(3, rows, C, seed=1) * 2 + 0.3).to(dtype)
    dy = rnd(3, rows, C, seed=2).to(dtype)
    xr = x.float().detach().clone().requires_grad_(True)
    ref(xr).backward(dy.float())
    xn = x.detach().clone().requires_grad_(True)
    yn = nat(xn)
    yn.backward(dy)
    tol = TOL[dtype]
    assert rel(yn, ref(x.float())) <= tol and rel(xn.grad, xr.grad) <= 2 * tol
    assert rel(nat.weight._pd_grad, ref.weight.grad) <= 2 * tol and rel(nat.bias._pd_grad, ref.bias.grad) <= 2 * tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("approx", ["tanh", "none"])
def test_gelu(dtype, approx):
    x = (rnd(7, 33, 40, seed=3) * 2).to(dtype)
    dy = rnd(7, 33, 40, seed=4).to(dtype)
    xr = x.float().detach().clone().requires_grad_(True)
    yr = F.gelu(xr, approximate=approx)
    yr.backward(dy.float())
    xn = x.detach().clone().requires_grad_(True)
    yn = layers.NativeGELU(approx)(xn)
    yn.backward(dy)
    assert rel(yn, yr) <= TOL[dtype] and rel(xn.grad, xr.grad) <= TOL[dtype]


@pytest.mark.parametrize("fp16", [False, True], ids=["fp32", "bf16"])
def test_gpt_two_stage_pipeline_2bw_matches_oracle(fp16):
    import pipeline_util as pu
    batch, n = 4, 8
    cfg = dict(layers=4, hidden=128, heads=4, seq_len=32, vocab=500, dropout=0.0)
    pkg = stages.gpt2(2, **cfg)
    conf = dict(pkg.conf, stage_to_depth_map=None)
    torch.manual_seed(0)
    omodel = pkg.model(torch.nn.CrossEntropyLoss())
    pipe_o = oracle.PipelineOracle(omodel, conf["module_to_stage_map"], conf["stage_to_rank_map"], None, "Adam",
                                   dict(lr=1e-3, weight_decay=0.0), macrobatch=True)
    data = lambda: stages.SyntheticTokens(batch, n, cfg["seq_len"], cfg["vocab"])
    pipe_o.run({0: data()}, n)
    ref_losses = pipe_o.ranks[1]["losses"]
    bs = pkg.boundary_shapes(batch)
    shapes = ({k: tuple(v) for k, v in bs.items()},
              {k: (torch.int64 if k in ("input0", "target") else torch.float32) for k in bs})
    pu.schedule.reset_local()
    torch.manual_seed(0)
    workers = [pu.make_worker(pkg, conf, rank, batch, fp16, pu.communication.LOCAL, shapes=shapes, lr=1e-3,
                              weight_decay=0.0, seed=0, optimizer="adam", macrobatch=True) for rank in range(2)]
    r0 = workers[0][0]
    blk = r0.modules()[0].parts[1]
    assert isinstance(blk.ln_1, layers.NativeLayerNorm) and isinstance(blk.act, layers.NativeGELU)
    assert isinstance(blk.attn.c_attn, layers.NativeLinear) and isinstance(r0.modules()[0].parts[0].wte, layers.NativeEmbedding)
    assert all(opt.num_versions == 2 for _, opt in workers[:1])      # 2BW: at most two weight versions
    pipe = pu.schedule.LocalPipeline(workers)
    r0.set_loader(data())
    workers[1][0].set_loader(None)
    losses = []
    pipe.run([n, n], on_loss=lambda k, i, rr: losses.append(float(rr.loss)))
    print("\n[%s] gpt 2-stage 2BW losses %s vs oracle %s" % ("bf16" if fp16 else "fp32", [round(v, 4) for v in losses],
                                                           [round(v, 4) for v in ref_losses]))
    tol = 2e-2 if fp16 else 1e-3
    assert len(losses) == n
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) <= tol * abs(b), (losses, ref_losses)
    if not fp16:
        for (r, _), st in zip(workers, pipe_o.ranks):
            sd = st["entries"][0][0].state_dict()
            for k, v in r.modules()[0].state_dict().items():
                # Adam's first steps are sign-like (g / sqrt(g^2)): an element whose gradient is near zero can move by
                # a fraction of lr either way, which is what these bounds allow for (weights ~0.02, lr 1e-3)
                assert rel(v.cpu(), sd[k]) <= (1e-2 if v.dim() >= 2 else 2e-2), k
    assert pf.gemm_poll_error() == 0


@pytest.mark.parametrize("B,H,T", [(2, 3, 128), (1, 2, 384), (2, 16, 512)])
def test_causal_attention_core_vs_torch(B, H, T):
    """The attention core on the tensor cores (batched contractions + causal softmax rows) against torch's
    scaled_dot_product_attention in fp32 on the same bf16 inputs, forward and gradient."""
    from pipedream_b200 import gpt_blocks
    d = 64
    C = H * d
    g = torch.Generator().manual_seed(5)
    qkv = (torch.randn(B, T, 3 * C, generator=g) * 0.8).cuda().to(torch.bfloat16)
    dout = torch.randn(B, T, C, generator=g).cuda().to(torch.bfloat16)
    core = gpt_blocks.CausalAttentionCore(H)
    ref_in = qkv.float().detach().clone().requires_grad_(True)
    ref = core(ref_in)
    ref.backward(dout.float())
    nat = layers.nativize(torch.nn.Sequential(gpt_blocks.CausalAttentionCore(H)))[0]
    assert isinstance(nat, layers.NativeCausalAttentionCore)
    x = qkv.detach().clone().requires_grad_(True)
    y = nat(x)
    y.backward(dout)
    assert nat.native_calls == 1
    print("attention core vs torch fp32: output %.2e, gradient %.2e" % (rel(y, ref), rel(x.grad, ref_in.grad)))
    assert rel(y, ref) <= 2e-2, rel(y, ref)
    assert rel(x.grad, ref_in.grad) <= 3e-2, rel(x.grad, ref_in.grad)
    # the three parts of the gradient separately (a wrong block would hide in the norm of the whole)
    gq, gk, gv = [x.grad.view(B, T, 3, C)[:, :, i] for i in range(3)]
    rq, rk, rv = [ref_in.grad.view(B, T, 3, C)[:, :, i] for i in range(3)]
    for name, a, b in (("dq", gq, rq), ("dk", gk, rk), ("dv", gv, rv)):
        assert rel(a, b) <= 3e-2, (name, rel(a, b))
    assert pf.gemm_poll_error() == 0
    # shapes the kernels are not written for run the original module
    small = torch.randn(2, 32, 3 * 4 * 32, generator=g).cuda().to(torch.bfloat16)
    nat2 = layers.NativeCausalAttentionCore(gpt_blocks.CausalAttentionCore(4))
    nat2(small)
    assert nat2.native_calls == 0
