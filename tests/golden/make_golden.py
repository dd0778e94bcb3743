"""Generates the golden fixtures in this directory by running the *reference* implementation.

Run where a checkout of the reference (msr-fiddle/pipedream) is available; pass its path with --ref or in
the PIPEDREAM_REFERENCE environment variable:

    python tests/golden/make_golden.py --ref <reference checkout> [--only routing|stashing|vgg16|gnmt]

It imports the reference's runtime/ modules unmodified and records what they compute:

  routing_golden.json   stage/rank/warm-up assignment (runtime/runtime.py:129-222) and the
                        replica routing sequences (runtime/communication.py:456-521,583-608)
                        for the stage/rank maps of the benchmark configurations
  stashing_golden.json  the weight-stashing truth table (runtime/tests/backprop/
                        sgd_with_stashing.py:57-70), per-stage version traces of the 1F1B loop
                        (runtime/optimizer.py), and a small SGD/Adam parameter trajectory
  gnmt_large_golden.json  3 minibatches of the 8+8-layer GNMT stage modules with LabelSmoothing and
                        AdamWithWeightStashing on CPU: losses, boundary-tensor and parameter checksums
  vgg16_cfg1_golden.json  20 minibatches of the 2-stage VGG-16 pipeline (cut after conv4_3) on two
                        gloo CPU ranks: per-minibatch loss, parameter checksums, version trace

Shims (monkey patches only; no reference file is modified or copied): `.cuda()` is the
identity, `torch.cuda.set_device` is a no-op, and the optimizer wrapper's in-place weight
swaps run under `torch.autograd._unsafe_preserve_version_counter`, which restores the
`.data` semantics of the PyTorch 1.1 the reference was written for.  The worker processes
run with `python -O` because the reference asserts `tensor.is_cuda`.
"""
import argparse
import importlib
import json
import os
import subprocess
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _shim_cpu():
    torch.Tensor.cuda = lambda self, *a, **k: self
    torch.nn.Module.cuda = lambda self, *a, **k: self
    torch.cuda.set_device = lambda *a, **k: None


def _import_reference(ref, domain="image_classification"):
    sys.path.insert(0, os.path.join(ref, "runtime"))
    sys.path.insert(0, os.path.join(ref, "runtime", domain))
    sys.dont_write_bytecode = True
    import optimizer as ref_optimizer

    def wrap(fn):
        def inner(self, *a, **k):
            params = tuple(p for m in self.modules for p in m.parameters())
            with torch.autograd._unsafe_preserve_version_counter(params):
                return fn(self, *a, **k)
        return inner
    ref_optimizer.OptimizerWithWeightStashing.set_params = wrap(ref_optimizer.OptimizerWithWeightStashing.set_params)
    ref_optimizer.OptimizerWithWeightStashing.step = wrap(ref_optimizer.OptimizerWithWeightStashing.step)
    return ref_optimizer


# ----------------------------------------------------------------------------- routing
ROUTING_CONFIGS = {
    # name: (number of model entries incl. criterion, module_to_stage_map, stage_to_rank_map, depth map)
    "cfg1_vgg16_2stage": (3, [0, 1, 1], {0: [0], 1: [1]}, None),
    "cfg2_vgg16_hybrid_3_1": (3, [0, 1, 1], {0: [0, 1, 2], 1: [3]}, {"0": 1, "1": 0}),
    "cfg2_vgg16_hybrid_3_1_nodepth": (3, [0, 1, 1], {0: [0, 1, 2], 1: [3]}, None),
    "cfg3_resnet50_8stage": (9, [0, 1, 2, 3, 4, 5, 6, 7, 7], {s: [s] for s in range(8)}, None),
    "cfg4_gnmt_4x2": (5, [0, 1, 2, 3, 3], {0: [0, 1], 1: [2, 3], 2: [4, 5], 3: [6, 7]}, None),
    "hybrid_7_1": (3, [0, 1, 1], {0: [0, 1, 2, 3, 4, 5, 6], 1: [7]}, None),
    "hybrid_6_2": (3, [0, 1, 1], {0: [0, 1, 2, 3, 4, 5], 1: [6, 7]}, None),
    "hybrid_2_4_1": (4, [0, 1, 2, 2], {0: [0, 1], 1: [2, 3, 4, 5], 2: [6]}, None),
    "hybrid_1_3": (3, [0, 1, 1], {0: [0], 1: [1, 2, 3]}, None),
    "dp_4": (2, [0, 0], {0: [0, 1, 2, 3]}, None),
}


def make_routing(ref):
    _shim_cpu()
    _import_reference(ref)
    import communication as ref_comm
    import runtime as ref_runtime

    class FakeHandler(ref_comm.CommunicationHandler):
        def __init__(self, **kw):        # no process group
            self.rank = kw["rank"]
            self.num_ranks_in_server = 1
            self.world_size = kw["world_size"]
            self.backend = "gloo"
            self.ranks_in_server = []

        def create_process_groups(self):
            pass

    ref_runtime.communication.CommunicationHandler = FakeHandler
    ref_runtime.dist.new_group = lambda ranks=None: None
    # DistributedDataParallel needs a process group; the stage arithmetic under test does not
    ref_runtime.torch.nn.parallel.DistributedDataParallel = lambda m, **k: m
    out = {}
    for name, (n_model, m2s, s2r, depth) in ROUTING_CONFIGS.items():
        world = sum(len(v) for v in s2r.values())
        per_rank = []
        for rank in range(world):
            # tiny stand-in model with the same tensor-name structure: one tensor per boundary
            names = ["input0"] + ["out%d" % i for i in range(n_model - 1)]
            model = [(torch.nn.Linear(2, 2), [names[i]], [names[i + 1]]) for i in range(n_model - 1)]
            model.append((torch.nn.MSELoss(), [names[-1]], ["loss"]))
            shapes = {n: (2, 2) for n in names}
            shapes["target"] = (2,)
            dtypes = {n: torch.float32 for n in names}
            dtypes["target"] = torch.int64
            r = ref_runtime.StageRuntime(
                model=model, distributed_backend="gloo", fp16=False, loss_scale=1,
                training_tensor_shapes=shapes, eval_tensor_shapes=dict(shapes),
                training_tensor_dtypes=dtypes, inputs_module_destinations={"input": 0},
                target_tensor_names={"target"},
                configuration_maps={"module_to_stage_map": m2s, "stage_to_rank_map": s2r,
                                    "stage_to_depth_map": depth},
                master_addr="127.0.0.1", rank=rank, local_rank=0, num_ranks_in_server=1,
                verbose_freq=0, model_type=ref_runtime.IMAGE_CLASSIFICATION)
            h = r.comm_handler
            rec = {
                "rank": rank, "stage": r.stage, "rank_in_stage": r.rank_in_stage,
                "num_ranks_in_stage": r.num_ranks_in_stage, "num_stages": r.num_stages,
                "num_ranks": r.num_ranks, "num_ranks_in_first_stage": r.num_ranks_in_first_stage,
                "num_warmup_minibatches": r.num_warmup_minibatches, "is_criterion": r.is_criterion,
                "ranks_in_previous_stage": list(r.ranks_in_previous_stage),
                "ranks_in_next_stage": list(r.ranks_in_next_stage),
                "send_ranks": {k: list(v) for k, v in r.send_ranks.items()},
                "receive_ranks": {k: list(v) for k, v in r.receive_ranks.items()},
                "tensor_tags": dict(r.tensor_tags),
                "messaging_schedule": [list(x) for x in h.messaging_schedule],
                "num_iterations_24": r.num_iterations(24) if (24 * r.num_ranks_in_first_stage) % r.num_ranks_in_stage == 0 else None,
                "adjusted_lr_0.1": r.get_adjusted_learning_rate(0.1),
            }
            # routing sequences over 24 minibatches
            fwd_recv, bwd_send, fwd_send, bwd_recv = [], [], [], []
            for mb in range(24):
                if r.num_ranks_in_previous_stage > 0:
                    fwd_recv.append(h.get_messaging_index(sending=False))
                    h.increment_messaging_index(sending=False)
                    bwd_send.append(h.get_messaging_index(sending=True))
                    h.increment_messaging_index(sending=True)
                if r.num_ranks_in_next_stage > 0:
                    n_next = r.num_ranks_in_next_stage
                    fwd_send.append((mb + r.rank_in_stage) % n_next)     # communication.py:606-607
                    bwd_recv.append((mb + r.rank_in_stage) % n_next)     # communication.py:586-587
            rec.update({"fwd_recv": fwd_recv, "bwd_send": bwd_send, "fwd_send": fwd_send, "bwd_recv": bwd_recv})
            per_rank.append(rec)
        out[name] = {"module_to_stage_map": m2s, "stage_to_rank_map": {str(k): v for k, v in s2r.items()},
                     "stage_to_depth_map": depth, "ranks": per_rank}
    with open(os.path.join(HERE, "routing_golden.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote routing_golden.json")


# ----------------------------------------------------------------------------- stashing
def _ref_version_trace(ref_sgd, num_warmup, n, macrobatch):
    """Drive the reference optimizer through the 1F1B loop of main_with_runtime.py:359-421 on a
    dummy model; the trace does not depend on data."""
    model = torch.nn.Linear(2, 2)
    opt = ref_sgd.SGDWithWeightStashing([model], list(model.parameters()), None, 1.0,
                                        num_versions=num_warmup + 1, lr=0.1, macrobatch=macrobatch)
    trace = []

    def fwd(i):
        trace.append(["F", i, opt.latest_version.version])

    def bwd(i):
        opt.zero_grad()
        opt.load_old_params()
        trace.append(["B", i, opt.current_version.version if opt.num_versions > 1 else opt.latest_version.version])
        for p in model.parameters():
            if p.grad is None:
                p.grad = torch.ones_like(p)
        opt.load_new_params()
        opt.step()
        trace.append(["S", i, opt.latest_version.version])

    for i in range(num_warmup):
        fwd(i)
    for i in range(n - num_warmup):
        fwd(num_warmup + i)
        bwd(i)
    for i in range(num_warmup):
        bwd(n - num_warmup + i)
    return trace


def make_stashing(ref):
    _shim_cpu()
    _import_reference(ref)
    import sgd as ref_sgd
    import adam as ref_adam
    out = {}
    # truth table of runtime/tests/backprop/sgd_with_stashing.py (current constructor signature)
    table = {}
    for k in (1, 2, 3):
        torch.manual_seed(7)
        N, D_in, D_H, D_out = 4, 4, 4, 4
        x1 = torch.randn(N, D_in).requires_grad_(True)
        y1 = torch.randn(N, D_out)
        xs = [x1, x1.clone().detach().requires_grad_(True), x1.clone().detach().requires_grad_(True)]
        model = torch.nn.Sequential(torch.nn.Linear(D_in, D_H), torch.nn.ReLU(), torch.nn.Linear(D_H, D_out))
        init = {k_: v.clone().tolist() for k_, v in model.state_dict().items()}
        loss_fn = torch.nn.MSELoss()
        opt = ref_sgd.SGDWithWeightStashing([model], list(model.parameters()), None, 1.0, num_versions=k, lr=1e-1)
        preds = [model(x) for x in xs]
        losses = [loss_fn(p, y1) for p in preds]
        grads = []
        for loss, x in zip(losses, xs):
            opt.zero_grad()
            opt.load_old_params()
            loss.backward()
            grads.append(x.grad.clone())
            opt.load_new_params()
            opt.step()
        table[str(k)] = {
            "equal_01": bool(torch.equal(grads[0], grads[1])), "equal_02": bool(torch.equal(grads[0], grads[2])),
            "latest_version": opt.latest_version.version, "current_version": opt.current_version.version,
            "x": x1.detach().tolist(), "y": y1.tolist(), "init": init,
            "x_grads": [g.tolist() for g in grads],
            "final": {k_: v.tolist() for k_, v in model.state_dict().items()},
        }
    out["truth_table"] = table
    traces = {}
    for w in (0, 1, 2, 3, 7):
        for macro in (False, True):
            traces["w%d_macro%d" % (w, int(macro))] = _ref_version_trace(ref_sgd, w, 12, macro)
    out["version_traces_n12"] = traces
    # optimizer trajectories on a fixed gradient sequence (values pin the update formulas)
    traj = {}
    for name, make in (("sgd", lambda m: ref_sgd.SGDWithWeightStashing([m], list(m.parameters()), None, 1.0, num_versions=2,
                                                                       lr=0.05, momentum=0.9, weight_decay=5e-4)),
                       ("adam", lambda m: ref_adam.AdamWithWeightStashing([m], list(m.parameters()), None, 1.0, num_versions=2,
                                                                          lr=2e-3, weight_decay=1e-4))):
        torch.manual_seed(11)
        m = torch.nn.Linear(8, 8)
        init = {k_: v.clone().tolist() for k_, v in m.state_dict().items()}
        opt = make(m)
        g = torch.Generator().manual_seed(12)
        steps = []
        for s in range(4):
            opt.zero_grad()
            opt.load_old_params()
            for p in m.parameters():
                p.grad = torch.randn(p.shape, generator=g)
            opt.load_new_params()
            opt.step()
            steps.append({k_: v.clone().tolist() for k_, v in m.state_dict().items()})
        traj[name] = {"init": init, "after_step": steps}
    out["trajectories"] = traj
    with open(os.path.join(HERE, "stashing_golden.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote stashing_golden.json")


# ----------------------------------------------------------------------------- VGG-16 config 1
def tensor_checksum(t):
    t = t.detach().double().flatten()
    k = min(8, t.numel())
    idx = torch.tensor([(j * (t.numel() - 1)) // max(1, k - 1) for j in range(k)], dtype=torch.long)
    return {"sum": t.sum().item(), "abs_sum": t.abs().sum().item(), "sq_sum": (t * t).sum().item(),
            "samples": t[idx].tolist()}


def vgg16_worker(ref, rank, steps, batch, out_path):
    _shim_cpu()
    _import_reference(ref)
    import runtime as ref_runtime
    import sgd as ref_sgd
    torch.manual_seed(0)
    module = importlib.import_module("models.vgg16.gpus=8")
    criterion = torch.nn.CrossEntropyLoss()
    model = module.model(criterion)
    for (m, _, _) in model[:-1]:
        for sub in m.modules():
            if isinstance(sub, torch.nn.Dropout):
                sub.p = 0.0            # CPU and GPU random streams differ; parity runs disable dropout
    shapes = {"input0": [batch, 3, 224, 224], "target": [batch]}
    dtypes = {"input0": torch.int64, "target": torch.int64}
    for (stage, inputs, outputs) in model[:-1]:
        ins = [torch.zeros(tuple(shapes[i]), dtype=torch.float32) for i in inputs]
        with torch.no_grad():
            o = stage(*ins)
        shapes[outputs[0]] = list(o.size())
        dtypes[outputs[0]] = o.dtype
    shapes = {k: tuple(v) for k, v in shapes.items()}
    conf = {"module_to_stage_map": [0, 1, 1], "stage_to_rank_map": {0: [0], 1: [1]}, "stage_to_depth_map": None}
    r = ref_runtime.StageRuntime(
        model=model, distributed_backend="gloo", fp16=False, loss_scale=1,
        training_tensor_shapes=shapes, eval_tensor_shapes=dict(shapes), training_tensor_dtypes=dtypes,
        inputs_module_destinations={"input": 0}, target_tensor_names={"target"}, configuration_maps=conf,
        master_addr="127.0.0.1", rank=rank, local_rank=rank, num_ranks_in_server=1, verbose_freq=0,
        model_type=ref_runtime.IMAGE_CLASSIFICATION)
    opt = ref_sgd.SGDWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1,
                                        num_versions=r.num_warmup_minibatches + 1, lr=0.01, momentum=0.9,
                                        weight_decay=5e-4)
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from pipedream_b200.stages import SyntheticImages
    n = steps
    r.train(n)
    r.set_loader(SyntheticImages(batch, n) if r.stage == 0 else None)
    losses, trace = [], []
    import time
    t0 = time.time()

    def bwd(i):
        opt.zero_grad()
        opt.load_old_params()
        trace.append(["B", i, opt.current_version.version if opt.num_versions > 1 else opt.latest_version.version])
        r.run_backward()
        opt.load_new_params()
        opt.step()

    w = r.num_warmup_minibatches
    for i in range(w):
        trace.append(["F", i, opt.latest_version.version])
        r.run_forward()
    for i in range(n - w):
        trace.append(["F", w + i, opt.latest_version.version])
        r.run_forward()
        if r.stage == r.num_stages - 1:
            losses.append(r.loss.item())
        bwd(i)
    for i in range(w):
        bwd(n - w + i)
    r.wait()
    elapsed = time.time() - t0
    params = {}
    for mi, m in enumerate(r.modules()):
        if isinstance(m, torch.nn.CrossEntropyLoss):
            continue
        for k, v in m.state_dict().items():
            params["module%d.%s" % (mi, k)] = tensor_checksum(v)
    with open(out_path, "w") as f:
        json.dump({"rank": rank, "stage": r.stage, "losses": losses, "trace": trace, "params": params,
                   "seconds": elapsed, "threads": torch.get_num_threads()}, f)


def make_vgg16(ref, steps=20, batch=8):
    procs, outs = [], []
    for rank in range(2):
        out_path = "/tmp/vgg16_cfg1_rank%d.json" % rank
        outs.append(out_path)
        env = dict(os.environ, OMP_NUM_THREADS=str(max(1, (os.cpu_count() or 2) // 2)), PYTHONDONTWRITEBYTECODE="1")
        procs.append(subprocess.Popen([sys.executable, "-O", os.path.abspath(__file__), "--ref", ref, "--worker",
                                       str(rank), "--steps", str(steps), "--batch", str(batch), "--out", out_path],
                                      env=env))
    for p in procs:
        if p.wait() != 0:
            raise RuntimeError("reference worker failed")
    ranks = [json.load(open(o)) for o in outs]
    gold = {
        "config": {"module": "models.vgg16.gpus=8", "batch": batch, "steps": steps, "lr": 0.01, "momentum": 0.9,
                   "weight_decay": 5e-4, "seed": 0, "data_seed": 1234, "dropout": "disabled (p=0) on both sides"},
        "losses": ranks[1]["losses"],
        "trace": {"stage0": ranks[0]["trace"], "stage1": ranks[1]["trace"]},
        "params": {"stage0": ranks[0]["params"], "stage1": ranks[1]["params"]},
        "reference_cpu_seconds": max(r["seconds"] for r in ranks),
        "reference_cpu_threads_per_rank": ranks[0]["threads"],
    }
    with open(os.path.join(HERE, "vgg16_cfg1_golden.json"), "w") as f:
        json.dump(gold, f, indent=1, sort_keys=True)
    print("wrote vgg16_cfg1_golden.json; reference took %.1f s" % gold["reference_cpu_seconds"])


# ----------------------------------------------------------------------------- GNMT (8+8 layers)
def make_gnmt(ref, steps=3, batch=8):
    """The reference's gnmt_large stage modules (4 stages run back to back in one process), its
    LabelSmoothing criterion and AdamWithWeightStashing, on CPU.  The reference's pack_utils CUDA
    extension does not build against current PyTorch; a pure-torch stand-in with the semantics of
    csrc/pack_utils_kernel.cu:24-63 and pack_utils.cpp:13-31 is injected in its place."""
    import types
    _shim_cpu()
    _import_reference(ref, "translation")
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from pipedream_b200.gnmt_blocks import _revert_varlen_torch
    from pipedream_b200.stages import SyntheticTranslation
    stub, c = types.ModuleType("pack_utils"), types.ModuleType("pack_utils._C")
    c.revert_varlen_tensor = lambda x, lengths: _revert_varlen_torch(x, lengths)

    def set_mask_cpp(lengths):
        T = int(lengths[0])
        return (torch.arange(T).unsqueeze(1) < lengths.unsqueeze(0)).to(torch.uint8)
    c.set_mask_cpp = set_mask_cpp
    stub._C = c
    sys.modules["pack_utils"], sys.modules["pack_utils._C"] = stub, c
    import adam as ref_adam
    from seq2seq.train.smoothing import LabelSmoothing
    torch.manual_seed(0)
    module = importlib.import_module("models.gnmt_large.gpus=4")
    model = module.model(LabelSmoothing(0, 0.1))
    stages_ = [m for (m, _, _) in model[:-1]]
    for m in stages_:
        for sub in m.modules():
            if isinstance(sub, torch.nn.Dropout):
                sub.p = 0.0
    params = [p for m in stages_ for p in m.parameters()]
    opt = ref_adam.AdamWithWeightStashing(stages_, params, None, 1, num_versions=1, lr=2e-3, weight_decay=1e-4)
    losses, tensors0 = [], {}
    import time
    t0 = time.time()
    for step, ((src, src_len), (tgt, tgt_len)) in enumerate(SyntheticTranslation(batch, steps, min_len=4, max_len=10)):
        t = {"input0": src, "input1": torch.LongTensor(src_len), "input2": tgt[:-1],
             "target": tgt[1:].contiguous().view(-1)}
        for (m, ins, outs) in model:
            if outs == ["loss"]:
                t["loss"] = m(t[ins[0]], t["target"])
            else:
                o = m(*[t[n] for n in ins])
                o = o if isinstance(o, tuple) else (o,)
                for n, v in zip(outs, o):
                    t[n] = v
        opt.zero_grad()
        opt.load_old_params()
        t["loss"].backward()
        opt.load_new_params()
        opt.step()
        losses.append(float(t["loss"]))
        if step == 0:
            tensors0 = {k: tensor_checksum(v) for k, v in t.items() if k.startswith("out")}
    out = {"config": {"module": "models.gnmt_large.gpus=4", "batch": batch, "steps": steps, "min_len": 4, "max_len": 10,
                      "optimizer": "Adam lr 2e-3 wd 1e-4", "seed": 0, "data_seed": 4321, "smoothing": 0.1,
                      "dropout": "disabled (p=0)"},
           "losses": losses, "boundary_tensors_step0": tensors0,
           "params": {"stage%d.%s" % (i, k): tensor_checksum(v) for i, m in enumerate(stages_)
                      for k, v in m.state_dict().items() if v is not None and ("bidir" in k or "layer1." not in k and "layer2." not in k)},
           "reference_cpu_seconds": time.time() - t0}
    with open(os.path.join(HERE, "gnmt_large_golden.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote gnmt_large_golden.json; losses", losses, "in %.1f s" % out["reference_cpu_seconds"])


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("PIPEDREAM_REFERENCE"), required=os.environ.get("PIPEDREAM_REFERENCE") is None)
    ap.add_argument("--only", default=None)
    ap.add_argument("--worker", type=int, default=None)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    if a.worker is not None:
        vgg16_worker(a.ref, a.worker, a.steps, a.batch, a.out)
    else:
        if a.only in (None, "routing"):
            subprocess.check_call([sys.executable, "-O", "-c",
                                   "import sys; sys.path.insert(0, %r); import make_golden; make_golden.make_routing(%r)" % (HERE, a.ref)])
        if a.only in (None, "stashing"):
            subprocess.check_call([sys.executable, "-O", "-c",
                                   "import sys; sys.path.insert(0, %r); import make_golden; make_golden.make_stashing(%r)" % (HERE, a.ref)])
        if a.only in (None, "vgg16"):
            make_vgg16(a.ref, a.steps, a.batch)
        if a.only in (None, "gnmt"):
            subprocess.check_call([sys.executable, "-O", "-c",
                                   "import sys; sys.path.insert(0, %r); import make_golden; make_golden.make_gnmt(%r)" % (HERE, a.ref)])
