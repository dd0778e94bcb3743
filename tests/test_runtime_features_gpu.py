"""StageRuntime features beyond the plain training step, on the GPU: activation recompute, checkpoints
(the reference's format, runtime/image_classification/main_with_runtime.py:322-330,507-511 and
runtime/runtime.py:306-312, and the full version ring), and the forward-only path with its ack clock
(runtime/runtime.py:629-653, main_with_runtime.py:430-504).

Bars (dropout off): a recomputed or resumed run does the same arithmetic as the plain run, but weight-gradient sums
are combined over K slices with fp32 atomics whose order differs from launch to launch, so two runs of the SAME
program already differ in the last bits.  Losses must agree to 1e-5 relative (fp32) / 2e-3 (bf16, where a last-bit
difference can move a bf16 weight by one ulp), parameters to 1e-5 / 1e-2 of their scale.  Evaluation losses equal
the stage modules chained by hand on the same weights."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

from pipedream_b200 import stages, schedule, communication  # noqa: E402
from pipedream_b200 import functional as pf                # noqa: E402
import pipeline_util as pu                                 # noqa: E402

torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_tf32 = False


def rel_err(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def small_pipeline(fp16, **kw):
    pkg = stages.vgg16("gpus=8")
    conf = dict(pkg.conf)
    conf["stage_to_depth_map"] = None
    schedule.reset_local()
    shapes = pu.tensor_shapes(pkg.model(torch.nn.CrossEntropyLoss()), 4)
    workers = [pu.make_worker(pkg, conf, rank, 4, fp16, communication.LOCAL, shapes=shapes, num_ranks_in_server=2,
                              lr=0.01, **kw) for rank in range(2)]
    return schedule.LocalPipeline(workers)


def run_steps(pipe, n, seed):
    (r0, _), (r1, _) = pipe.workers
    r0.set_loader(stages.SyntheticImages(4, n, seed=seed))
    r1.set_loader(None)
    losses = []
    pipe.run([n, n], on_loss=lambda k, i, rr: losses.append(float(rr.loss)))
    torch.cuda.synchronize()
    return losses


def params_of(pipe):
    return [p.detach().float().clone() for (r, _) in pipe.workers for p in r.parameters()]


def spread(losses, want, params, want_params):
    """(largest relative loss difference, largest parameter difference relative to the tensor's scale)."""
    assert len(losses) == len(want)
    dl = max(abs(a - b) / max(1.0, abs(b)) for a, b in zip(losses, want))
    dp = max(((a - b).abs().max() / b.abs().max().clamp_min(1e-3)).item() for a, b in zip(params, want_params))
    return dl, dp


@pytest.fixture(autouse=True)
def deterministic_weight_gradients():
    """Split-K weight gradients add their parts with fp32 atomics in a varying order, and this un-normalised network
    amplifies a last-bit difference into a visible one within a few steps; the tests here compare whole runs, so
    they switch the split off (pf.set_deterministic) and can then ask for (near) equality."""
    prev = pf.set_deterministic(True)
    yield
    pf.set_deterministic(prev)


def same_run(losses, want, params, want_params, fp16, noise=(0.0, 0.0)):
    """Within the stated bar (the plain path's own run-to-run spread `noise` is asserted to be zero first)."""
    assert noise == (0.0, 0.0), "two plain runs differ in deterministic mode: %r" % (noise,)
    ltol, ptol = (2e-3, 1e-2) if fp16 else (1e-5, 1e-5)
    dl, dp = spread(losses, want, params, want_params)
    print("difference (loss, parameters):", (dl, dp))
    assert dl <= ltol, (dl, losses, want)
    assert dp <= ptol, dp


@pytest.mark.parametrize("fp16", [False, True], ids=["fp32", "bf16"])
def test_recompute_matches_plain_run(fp16):
    """Stage 0 drops its activations after the forward pass and rebuilds them, on the stashed weight version,
    just before its backward pass: same losses, same parameters (to the run-to-run spread of the plain path)."""
    base = small_pipeline(fp16)
    ref_losses = run_steps(base, 6, 11)
    ref_params = params_of(base)
    again = small_pipeline(fp16)
    noise = spread(run_steps(again, 6, 11), ref_losses, params_of(again), ref_params)
    rec = small_pipeline(fp16, enable_recompute=True)
    assert rec.workers[0][0].enable_recompute and not rec.workers[1][0].enable_recompute
    losses = run_steps(rec, 6, 11)
    same_run(losses, ref_losses, params_of(rec), ref_params, fp16, noise)
    assert pf.gemm_poll_error() == 0


def test_recompute_keeps_only_stage_inputs():
    rec = small_pipeline(True, enable_recompute=True)
    r0 = rec.workers[0][0]
    r0.train(1)
    r0.set_loader(stages.SyntheticImages(4, 1, seed=3))
    r0.run_forward()
    kept = r0.tensors[-1]
    assert set(kept) == {"input0", "target", "_replay"}, sorted(kept)


def test_reference_format_checkpoint_fp32():
    """state_dict() of the runtime ("module<i>" keys) and of the optimizer, loaded into a fresh process image:
    training continues exactly as if it had not been interrupted (single stage, so no versions in flight)."""
    pkg = stages.vgg16("gpus=1")

    def fresh():
        return pu.make_worker(pkg, None, None, 4, False, None, lr=0.01)

    def steps(r, opt, n, seed):
        r.train(n)
        r.set_loader(stages.SyntheticImages(4, n, seed=seed))
        out = []
        schedule.train_1f1b(r, opt, n, on_forward=lambda i, rr: out.append(float(rr.loss)))
        return out

    # run-to-run spread of the uninterrupted six steps
    ra, oa = fresh()
    la = steps(ra, oa, 3, 5) + steps(ra, oa, 3, 6)
    rb, ob = fresh()
    lb = steps(rb, ob, 3, 5) + steps(rb, ob, 3, 6)
    noise = spread(lb, la, [p.detach() for p in rb.parameters()], [p.detach() for p in ra.parameters()])
    print("run-to-run spread (loss, parameters):", noise)
    del ra, oa, rb, ob

    r, opt = fresh()
    steps(r, opt, 3, 5)
    ckpt = {"state_dict": copy.deepcopy(r.state_dict()), "optimizer": copy.deepcopy(opt.state_dict())}
    assert sorted(ckpt["state_dict"]) == ["module%d" % i for i in range(len(r.modules()))]
    want = steps(r, opt, 3, 6)
    want_params = [p.detach().clone() for p in r.parameters()]
    # the order of the reference's driver: load the modules, build the optimizer, load its state
    torch.manual_seed(123)
    r2, _ = fresh()
    r2.load_state_dict(ckpt["state_dict"])
    from pipedream_b200 import sgd
    opt2 = sgd.SGDWithWeightStashing(r2.modules(), r2.master_parameters, r2.model_parameters, 1, num_versions=1,
                                     lr=0.01, momentum=0.9, weight_decay=5e-4)
    opt2.load_state_dict(ckpt["optimizer"])
    got = steps(r2, opt2, 3, 6)
    same_run(got, want, [p.detach() for p in r2.parameters()], want_params, False, noise)
    # and the other order: an optimizer that already holds the parameters is re-seeded by the load
    torch.manual_seed(321)
    r3, opt3 = fresh()
    r3.load_state_dict(ckpt["state_dict"])
    opt3.load_state_dict(ckpt["optimizer"])
    same_run(steps(r3, opt3, 3, 6), want, [p.detach() for p in r3.parameters()], want_params, False, noise)


def test_ring_checkpoint_mid_pipeline_bf16():
    """bf16 with fp32 master weights and two weight versions in flight on stage 0: the optimizer's ring state
    (every stashed version, the master copy, the counters) lets the run continue as if it had not stopped."""
    n1 = small_pipeline(True)
    l1 = run_steps(n1, 4, 21) + run_steps(n1, 4, 22)
    n2 = small_pipeline(True)
    l2 = run_steps(n2, 4, 21) + run_steps(n2, 4, 22)
    noise = spread(l2, l1, params_of(n2), params_of(n1))
    print("run-to-run spread (loss, parameters):", noise)
    del n1, n2
    a = small_pipeline(True)
    run_steps(a, 4, 21)
    saved = [(copy.deepcopy(r.state_dict()), copy.deepcopy(o.state_dict()), copy.deepcopy(o.ring_state_dict()))
             for (r, o) in a.workers]
    want = run_steps(a, 4, 22)
    want_params = params_of(a)
    torch.manual_seed(77)
    b = small_pipeline(True)
    for (r, o), (sd, osd, ring) in zip(b.workers, saved):
        r.load_state_dict(sd)
        o.load_state_dict(osd)
        o.load_ring_state_dict(ring)
    got = run_steps(b, 4, 22)
    same_run(got, want, params_of(b), want_params, True, noise)


def test_forward_only_with_ack_clock():
    """eval(): forward passes only, an ack flowing back per minibatch; the loss equals the stage modules chained
    by hand on the same weights and inputs."""
    pipe = small_pipeline(False)
    (r0, _), (r1, _) = pipe.workers
    n = 3
    loader = stages.SyntheticImages(4, n, seed=9)
    batches = list(loader)
    for r in (r0, r1):
        r.eval(n)
    r0.set_loader(loader)
    r1.set_loader(None)
    got = []
    with torch.no_grad():
        for _ in range(n):
            r0.run_forward()
            r1.run_forward()
            got.append(float(r1.loss))
            r1.run_ack()
            r0.run_ack()
    r0.wait(); r1.wait()
    assert "ack" in r0.send_ranks and "ack" in r1.receive_ranks
    assert r0.backward_minibatch_id == n and r1.backward_minibatch_id == n
    mods0, mods1 = r0.modules(), r1.modules()
    with torch.no_grad():
        for (x, y), g in zip(batches, got):
            h = x.cuda()
            for m in mods0:
                h = m(h)
            for m in mods1[:-1]:
                h = m(h)
            want = float(mods1[-1](h, y.cuda()))
            assert abs(want - g) <= 1e-6 * max(1.0, abs(want)), (want, g)
    # the epoch after an evaluation trains again ("ack" leaves the rank maps)
    for r in (r0, r1):
        r.train(1)
    assert "ack" not in r0.send_ranks and "ack" not in r1.receive_ranks


@pytest.mark.parametrize("fp16", [False, True], ids=["fp32", "bf16"])
def test_accumulation_over_more_than_two_microbatches(fp16):
    """`update_interval` (an extension beside the reference's `macrobatch`, whose accumulation length is the
    version count capped at two, runtime/optimizer.py:36-52): k micro-batches accumulate into the fp32 gradient
    arena, one optimizer step follows the k-th with the gradients scaled by 1 / k, and two weight versions stay
    enough.  Checked against one step of torch SGD on the k micro-batches joined into one batch."""
    from pipedream_b200 import layers
    from pipedream_b200.stashing_optimizers import SGDWithWeightStashing
    k, mb, steps = 5, 16, 3
    torch.manual_seed(3)
    ref = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 32)).cuda()
    ours = layers.nativize(copy.deepcopy(ref))
    if fp16:
        ours = ours.to(torch.bfloat16)
    assert isinstance(ours[0], layers.NativeLinear)
    opt = SGDWithWeightStashing([ours], list(ours.parameters()), None, 1, num_versions=4, lr=0.05, momentum=0.9,
                                weight_decay=1e-4, macrobatch=True, update_interval=k)
    assert opt.num_versions == 2 and opt.update_interval == k
    with pytest.raises(ValueError):
        SGDWithWeightStashing([ours], list(ours.parameters()), None, 1, num_versions=2, lr=0.05, update_interval=3)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
    g = torch.Generator().manual_seed(11)
    for s in range(steps):
        xs = [torch.randn(mb, 64, generator=g).cuda() for _ in range(k)]
        ts = [torch.randn(mb, 32, generator=g).cuda() for _ in range(k)]
        ropt.zero_grad()
        (sum(((ref(x) - t) ** 2).mean() for x, t in zip(xs, ts)) / k).backward()
        ropt.step()
        for i, (x, t) in enumerate(zip(xs, ts)):
            opt.zero_grad()
            xin = x.to(torch.bfloat16) if fp16 else x
            ((ours(xin).float() - t) ** 2).mean().backward()
            before = opt.latest_version.version
            opt.step()
            assert opt.latest_version.version == before + (1 if i == k - 1 else 0)
    assert [e for e in opt.trace if e[0] == "step"] == [("step", v) for v in range(1, steps + 1)]
    tol = 3e-2 if fp16 else 2e-5
    for p, q in zip(ours.parameters(), ref.parameters()):
        assert rel_err(p.float(), q) <= tol
    assert pf.gemm_poll_error() == 0
