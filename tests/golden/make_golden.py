"""Generates the golden fixtures in this directory by running the *reference* implementation.

Run where a checkout of the reference (msr-fiddle/pipedream) is available; pass its path with --ref or in
the PIPEDREAM_REFERENCE environment variable:

    python tests/golden/make_golden.py --ref <reference checkout> [--only routing|stashing|vgg16|gnmt]

It imports the reference's runtime/ modules unmodified and records what they compute:

  partition_golden.json  stage cuts and replication factors the reference's partitioner (optimizer/
                        optimizer_graph_hierarchical.py) computes for eight synthetic chain profiles
  signatures_golden.json  constructor / method signatures of the runtime and optimizer classes the driver scripts use
  routing_golden.json   stage/rank/warm-up assignment (runtime/runtime.py:129-222) and the
                        replica routing sequences (runtime/communication.py:456-521,583-608)
                        for the stage/rank maps of the benchmark configurations
  stashing_golden.json  the weight-stashing truth table (runtime/tests/backprop/
                        sgd_with_stashing.py:57-70), per-stage version traces of the 1F1B loop
                        (runtime/optimizer.py), and a small SGD/Adam parameter trajectory
  gnmt_pipeline_golden.json  20 minibatches of the same stage modules as the reference's real 4-stage pipeline: the
                        reference runtime in translation mode on four gloo CPU ranks, sorted variable-length
                        batches, AdamWithWeightStashing with 4..1 weight versions: losses, version traces, parameters
  gnmt_large_golden.json  3 minibatches of the 8+8-layer GNMT stage modules with LabelSmoothing and
                        AdamWithWeightStashing on CPU: losses, boundary-tensor and parameter checksums
  vgg16_cfg1_golden.json  20 minibatches of the 2-stage VGG-16 pipeline (cut after conv4_3) on two
                        gloo CPU ranks: per-minibatch loss, parameter checksums, version trace
  vgg16_cfg1_f64_golden.json  the same run with the reference modules in float64 (arbitrates fp32 deviations)
  resnet50_gpus4_golden.json  the reference's 3-stage ResNet-50 package (models.resnet50.gpus=4; two tensors
                        cross each boundary): a description of every stage recorded from the live modules
                        (declarations from named_children, dataflow from a torch.fx trace) and 6 minibatches
                        of the pipeline on three gloo CPU ranks with BatchNorm in training mode

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
    _shim_batchnorm()


def _shim_batchnorm():
    """In a pipelined stage the forward pass of minibatch i+1 runs before the backward pass of minibatch i and
    moves BatchNorm's running statistics in place.  Current PyTorch saves those buffers with the autograd graph
    and refuses the delayed backward ("modified by an inplace operation"); the PyTorch 1.1 the reference was
    written for did not.  The stand-in computes the same function - normalisation by the batch statistics - with
    the running statistics kept out of the graph and updated by the same formula (momentum, unbiased variance)."""
    import torch.nn.functional as F

    def forward(self, x):
        if not self.training or not self.track_running_stats:
            return F.batch_norm(x, self.running_mean, self.running_var, self.weight, self.bias, self.training, 0.0, self.eps)
        y = F.batch_norm(x, None, None, self.weight, self.bias, True, 0.0, self.eps)
        with torch.no_grad():
            dims = [0] + list(range(2, x.dim()))
            m = self.momentum
            self.running_mean.mul_(1 - m).add_(x.mean(dims), alpha=m)
            self.running_var.mul_(1 - m).add_(x.var(dims, unbiased=True), alpha=m)
            self.num_batches_tracked += 1
        return y
    torch.nn.BatchNorm2d.forward = forward


def _shim_transport(ref_comm, float64=False):
    """gloo in current PyTorch refuses non-contiguous tensors (the GNMT stages send transposed views); and the
    reference marks a received activation as requiring a gradient only when it is float32
    (runtime/communication.py:595-596), so a float64 run needs the same mark for float64."""
    import torch.distributed as dist
    orig_send = dist.send

    def send(tensor, dst=None, group=None, tag=0, **kw):
        return orig_send(tensor.contiguous(), dst=dst, group=group, tag=tag, **kw)
    dist.send = send
    ref_comm.dist.send = send
    if float64:
        orig_recv = ref_comm.CommunicationHandler.recv

        def recv(self, tensor_name, forward_minibatch_id, backward_minibatch_id, backward=False):
            t = orig_recv(self, tensor_name, forward_minibatch_id, backward_minibatch_id, backward=backward)
            if not backward and t.dtype == torch.float64:
                t = t.requires_grad_()
            return t
        ref_comm.CommunicationHandler.recv = recv


def _import_reference(ref, domain="image_classification"):
    sys.path.insert(0, os.path.join(ref, "runtime"))
    sys.path.insert(0, os.path.join(ref, "runtime", domain))
    sys.dont_write_bytecode = True
    import optimizer as ref_optimizer

    def wrap(fn):
        import functools

        @functools.wraps(fn)
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


# ----------------------------------------------------------------------------- interface
def make_signatures(ref):
    """Constructor and method signatures of the classes main_with_runtime.py uses, read off the imported reference."""
    import inspect
    _shim_cpu()
    _import_reference(ref)
    import runtime as ref_runtime
    import sgd as ref_sgd
    import adam as ref_adam
    import optimizer as ref_optimizer

    def sig(fn):
        out = []
        for name, p in inspect.signature(fn).parameters.items():
            if name == "self":
                continue
            out.append([name, None if p.default is inspect.Parameter.empty else repr(p.default)])
        return out

    def methods(cls, names):
        return {n: sig(getattr(cls, n)) for n in names}
    out = {
        "runtime.StageRuntime": methods(ref_runtime.StageRuntime, [
            "__init__", "train", "eval", "set_loader", "run_forward", "run_backward", "run_ack", "wait", "num_iterations",
            "get_adjusted_learning_rate", "state_dict", "load_state_dict", "modules", "parameters", "zero_grad", "cuda",
            "num_tokens", "initialize", "receive_tensors_forward", "send_tensors_forward", "receive_tensors_backward",
            "send_tensors_backward"]),
        "runtime.constants": {k: getattr(ref_runtime, k) for k in ("IMAGE_CLASSIFICATION", "TRANSLATION", "SPEECH_TO_TEXT")},
        "sgd.SGDWithWeightStashing": methods(ref_sgd.SGDWithWeightStashing, ["__init__"]),
        "adam.AdamWithWeightStashing": methods(ref_adam.AdamWithWeightStashing, ["__init__"]),
        "optimizer.OptimizerWithWeightStashing": methods(ref_optimizer.OptimizerWithWeightStashing, [
            "__init__", "initialize_queue", "get_params", "set_params", "load_old_params", "load_new_params", "zero_grad",
            "step"]),
    }
    with open(os.path.join(HERE, "signatures_golden.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote signatures_golden.json")


# ----------------------------------------------------------------------------- partitioner
def make_partition(ref):
    """The reference's own `compute_partitioning` + `analyze_partitioning` on synthetic chain profiles."""
    import random
    import types
    sys.modules.setdefault("graphviz", types.ModuleType("graphviz"))
    sys.path.insert(0, ref)
    sys.path.insert(0, os.path.join(ref, "optimizer"))
    import optimizer_graph_hierarchical as ogh
    cases = []
    for seed, L, machines, straight, ratio in ((1, 12, 4, False, None), (2, 16, 8, False, None), (3, 10, 4, True, None),
                                               (4, 14, 8, False, 1.0), (5, 9, 3, False, 1.0), (6, 20, 8, True, 1.0),
                                               (7, 16, 6, False, None), (8, 13, 8, False, 2.0)):
        rnd = random.Random(seed)
        times = [rnd.uniform(0.5, 8.0) * (3.0 if rnd.random() < 0.2 else 1.0) for _ in range(L)]
        params = [rnd.choice([0.0, 1e6, 5e7, 5e8, 3e9]) for _ in range(L)]
        acts = [rnd.uniform(1e5, 5e7) for _ in range(L)]
        outs = [rnd.uniform(1e5, 3e7) for _ in range(L)]
        bandwidth = rnd.choice([2e8, 1e9, 5e9])
        ogh.straight_pipeline = straight
        ogh.use_memory_constraint = False
        ogh.memory_size = 1e18
        ogh.use_fewer_machines = False
        ogh.activation_compression_ratio = ratio
        states = []
        ct = ps = ac = 0.0
        for i in range(L):
            ct += times[i]; ps += params[i]; ac += acts[i]
            states.append(types.SimpleNamespace(compute_time=ct, parameter_size=ps, activation_size=ac,
                                                output_activation_size=outs[i], antichain=[i]))
        compute_times, activation_sizes, parameter_sizes = [], [], []
        for i in range(L + 1):
            r1, r2, r3 = [], [], []
            for j in range(L):
                if i == 0:
                    r1.append(states[j].compute_time); r2.append(states[j].activation_size); r3.append(states[j].parameter_size)
                elif j > i - 1:
                    r1.append(states[j].compute_time - states[i - 1].compute_time)
                    r2.append(states[j].activation_size - states[i - 1].activation_size)
                    r3.append(states[j].parameter_size - states[i - 1].parameter_size)
                else:
                    r1.append(None); r2.append(None); r3.append(None)
            compute_times.append(r1); activation_sizes.append(r2); parameter_sizes.append(r3)
        preds = [list(range(j)) for j in range(L)]
        A = ogh.compute_partitioning(compute_times, activation_sizes, parameter_sizes, outs, preds, machines, 1, bandwidth,
                                     final_level=True)
        # replication factors are not returned by analyze_partitioning: walk the table the same way
        splits = ogh.analyze_partitioning(A, states, 0, L, bandwidth, machines, ratio, False, False)
        meta = A[0][L - 1][machines - 1]
        reps, nxt = [], meta[1]
        while nxt is not None:
            reps.append(meta[2])
            meta = A[0][nxt[0]][nxt[1]]
            nxt = meta[1]
        reps.append(meta[2])
        reps.reverse()
        cases.append({"times": times, "param_bytes": params, "act_bytes": acts, "out_bytes": outs, "bandwidth": bandwidth,
                      "num_machines": machines, "straight": straight, "compression_ratio": ratio,
                      "splits": splits, "replication": reps, "pipeline_time": A[0][L - 1][machines - 1][0]})
    with open(os.path.join(HERE, "partition_golden.json"), "w") as f:
        json.dump(cases, f, indent=1)
    print("wrote partition_golden.json:", [(c["splits"], c["replication"]) for c in cases])


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


PIPELINES = {
    # name: (module, module_to_stage_map, ranks, lr, momentum, weight_decay)
    "vgg16": ("models.vgg16.gpus=8", [0, 1, 1], 2, 0.01, 0.9, 5e-4),
    "resnet50": ("models.resnet50.gpus=4", [0, 1, 2, 2], 3, 0.01, 0.9, 1e-4),
}


def vgg16_worker(ref, rank, steps, batch, out_path, which="vgg16", f64=False):
    _shim_cpu()
    _import_reference(ref)
    import runtime as ref_runtime
    import sgd as ref_sgd
    import communication as ref_comm
    _shim_transport(ref_comm, float64=f64)
    torch.manual_seed(0)
    mod_name, m2s, world, lr, momentum, wd = PIPELINES[which]
    module = importlib.import_module(mod_name)
    criterion = torch.nn.CrossEntropyLoss()
    model = module.model(criterion)
    if f64:
        model = [(m.double() if i < len(model) - 1 else m, a, b) for i, (m, a, b) in enumerate(model)]
    fdt = torch.float64 if f64 else torch.float32
    for (m, _, _) in model[:-1]:
        for sub in m.modules():
            if isinstance(sub, torch.nn.Dropout):
                sub.p = 0.0            # CPU and GPU random streams differ; parity runs disable dropout
    shapes = {"input0": [batch, 3, 224, 224], "target": [batch]}
    dtypes = {"input0": torch.int64, "target": torch.int64}
    for (stage, inputs, outputs) in model[:-1]:
        ins = [torch.zeros(tuple(shapes[i]), dtype=fdt) for i in inputs]
        was_training = stage.training
        stage.eval()                       # the dry run must not move BatchNorm's running statistics
        with torch.no_grad():
            o = stage(*ins)
        stage.train(was_training)
        o = o if isinstance(o, tuple) else (o,)
        for name, t in zip(outputs, o):
            shapes[name] = list(t.size())
            dtypes[name] = t.dtype
    shapes = {k: tuple(v) for k, v in shapes.items()}
    conf = {"module_to_stage_map": m2s, "stage_to_rank_map": {s: [s] for s in range(world)}, "stage_to_depth_map": None}
    r = ref_runtime.StageRuntime(
        model=model, distributed_backend="gloo", fp16=False, loss_scale=1,
        training_tensor_shapes=shapes, eval_tensor_shapes=dict(shapes), training_tensor_dtypes=dtypes,
        inputs_module_destinations={"input": 0}, target_tensor_names={"target"}, configuration_maps=conf,
        master_addr="127.0.0.1", rank=rank, local_rank=rank, num_ranks_in_server=1, verbose_freq=0,
        model_type=ref_runtime.IMAGE_CLASSIFICATION)
    opt = ref_sgd.SGDWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1,
                                        num_versions=r.num_warmup_minibatches + 1, lr=lr, momentum=momentum,
                                        weight_decay=wd)
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from pipedream_b200.stages import SyntheticImages
    n = steps
    r.train(n)
    data = SyntheticImages(batch, n)
    if f64:
        data = [(x.double(), y) for (x, y) in data]
    r.set_loader(data if r.stage == 0 else None)
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


def _wait_all(procs, limit_s):
    """Waits for every worker; as soon as one fails (or the limit passes) the others are killed - a rank that
    died leaves its peers blocked in a receive for ever."""
    import time
    t0 = time.time()
    while True:
        codes = [p.poll() for p in procs]
        if all(c == 0 for c in codes):
            return
        if any(c not in (None, 0) for c in codes) or time.time() - t0 > limit_s:
            for p in procs:
                if p.poll() is None:
                    p.kill()
            raise RuntimeError("reference worker failed or timed out (exit codes %s)" % codes)
        time.sleep(1.0)


def run_pipeline(ref, which, steps, batch, f64=False):
    """The reference runtime on one gloo CPU rank per stage; returns the per-rank records."""
    world = PIPELINES[which][2]
    procs, outs = [], []
    for rank in range(world):
        out_path = "/tmp/%s_rank%d.json" % (which, rank)
        outs.append(out_path)
        env = dict(os.environ, OMP_NUM_THREADS=str(max(1, (os.cpu_count() or 2) // world)), PYTHONDONTWRITEBYTECODE="1")
        cmd = [sys.executable, "-O", os.path.abspath(__file__), "--ref", ref, "--worker", str(rank), "--steps", str(steps),
               "--batch", str(batch), "--out", out_path, "--pipeline", which]
        procs.append(subprocess.Popen(cmd + (["--f64"] if f64 else []), env=env))
    _wait_all(procs, 1500)
    return [json.load(open(o)) for o in outs]


def make_vgg16(ref, steps=20, batch=8, f64=False):
    ranks = run_pipeline(ref, "vgg16", steps, batch, f64)
    gold = {
        "config": {"module": "models.vgg16.gpus=8", "batch": batch, "steps": steps, "lr": 0.01, "momentum": 0.9,
                   "weight_decay": 5e-4, "seed": 0, "data_seed": 1234, "dropout": "disabled (p=0) on both sides"},
        "losses": ranks[1]["losses"],
        "trace": {"stage0": ranks[0]["trace"], "stage1": ranks[1]["trace"]},
        "params": {"stage0": ranks[0]["params"], "stage1": ranks[1]["params"]},
        "reference_cpu_seconds": max(r["seconds"] for r in ranks),
        "reference_cpu_threads_per_rank": ranks[0]["threads"],
    }
    name = "vgg16_cfg1_f64_golden.json" if f64 else "vgg16_cfg1_golden.json"
    if f64:
        gold["config"]["dtype"] = "float64"
    with open(os.path.join(HERE, name), "w") as f:
        json.dump(gold, f, indent=1, sort_keys=True)
    print("wrote %s; reference took %.1f s" % (name, gold["reference_cpu_seconds"]))


# ----------------------------------------------------------------------------- ResNet-50, 3 stages
def describe_stage(stage):
    """Declarations and dataflow of a live stage module, in the form pipedream_b200.stages.SpecStage takes."""
    import torch.fx
    import operator
    mods = []
    for name, m in stage.named_children():
        kind = type(m).__name__
        if kind == "Conv2d":
            kw = {"in_channels": m.in_channels, "out_channels": m.out_channels, "kernel_size": list(m.kernel_size),
                  "stride": list(m.stride), "padding": list(m.padding), "bias": m.bias is not None}
        elif kind == "BatchNorm2d":
            kw = {"num_features": m.num_features, "eps": m.eps, "momentum": m.momentum, "affine": m.affine,
                  "track_running_stats": m.track_running_stats}
        elif kind == "ReLU":
            kw = {"inplace": m.inplace}
        elif kind == "MaxPool2d":
            kw = {"kernel_size": m.kernel_size, "stride": m.stride, "padding": m.padding, "dilation": m.dilation,
                  "ceil_mode": m.ceil_mode}
        elif kind == "AvgPool2d":
            kw = {"kernel_size": m.kernel_size, "stride": m.stride, "padding": m.padding}
        elif kind == "Linear":
            kw = {"in_features": m.in_features, "out_features": m.out_features, "bias": m.bias is not None}
        elif kind == "Dropout":
            kw = {"p": m.p}
        elif kind == "Embedding":
            kw = {"num_embeddings": m.num_embeddings, "embedding_dim": m.embedding_dim, "padding_idx": m.padding_idx}
        elif kind == "LSTM":
            assert m.num_layers == 1 and not m.bidirectional
            kw = {"input_size": m.input_size, "hidden_size": m.hidden_size}
        elif kind == "EmuBidirLSTM":
            kw = {"input_size": m.bidir.input_size, "hidden_size": m.bidir.hidden_size}
        elif kind == "RecurrentAttention":
            # (constructor order input, context, hidden; seq2seq/models/decoder.py:13-24)
            kw = {"input_size": m.rnn.input_size, "context_size": m.attn.linear_k.in_features, "hidden_size": m.rnn.hidden_size}
        elif kind == "Classifier":
            kw = {"in_features": m.classifier.in_features, "out_features": m.classifier.out_features}
        else:
            raise ValueError("unexpected module type %s" % kind)
        mods.append([name, kind, kw])

    class _LeafTracer(torch.fx.Tracer):
        def is_leaf_module(self, m, qualname):
            return True
    g = _LeafTracer().trace(stage)
    flow, returns, n_in = [], [], 0

    def arg_name(a):
        return a.name if isinstance(a, torch.fx.Node) else a
    none_names = {}
    for node in g.nodes:
        if node.op == "placeholder":
            flow.append([node.name, "input", n_in])
            n_in += 1
        elif node.op == "call_module":
            args = []
            for a in node.args:
                if a is None:                       # `outK = None` in the generated source: a statement of its own
                    nm = "none_%d" % len(none_names)
                    none_names[nm] = True
                    flow.append([nm, "none"])
                    args.append(nm)
                else:
                    args.append(a.name)
            flow.append([node.name, node.target] + args)
        elif node.op == "call_function" and node.target is operator.getitem:
            flow.append([node.name, "getitem", node.args[0].name, node.args[1]])
        elif node.op == "call_function" and node.target is torch.cat:
            flow.append([node.name, "cat", node.args[1]] + [a.name for a in node.args[0]])
        elif node.op == "call_method" and node.target == "clone":
            flow.append([node.name, "clone", node.args[0].name])
        elif node.op == "call_method" and node.target == "size":
            assert node.args[1] == 0
            flow.append([node.name, "size0", node.args[0].name])
        elif node.op == "call_method" and node.target == "view":
            assert node.args[2] == -1
            flow.append([node.name, "flatten", node.args[0].name, node.args[1].name])
        elif node.op == "call_function" and node.target in (operator.add, torch.add):
            flow.append([node.name, "add", node.args[0].name, node.args[1].name])
        elif node.op == "output":
            res = node.args[0]
            returns = [r.name for r in (res if isinstance(res, (tuple, list)) else (res,))]
        else:
            raise ValueError("unexpected node %s %s" % (node.op, node.target))
    return {"modules": mods, "flow": flow, "returns": returns}


def make_resnet50(ref, steps=6, batch=8):
    _shim_cpu()
    _import_reference(ref)
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from pipedream_b200 import stages as pd_stages
    torch.manual_seed(0)
    module = importlib.import_module("models.resnet50.gpus=4")
    model = module.model(torch.nn.CrossEntropyLoss())
    desc = {"arch": module.arch(), "stages": []}
    for (m, ins, outs) in model[:-1]:
        d = describe_stage(m)
        d["inputs"], d["outputs"] = list(ins), list(outs)
        desc["stages"].append(d)
    # the description rebuilds the package bit for bit under the same seed
    torch.manual_seed(0)
    mine = pd_stages.SpecPackage(desc).model(torch.nn.CrossEntropyLoss())
    for (a, _, _), (b, _, _) in zip(model[:-1], mine[:-1]):
        sa, sb = a.state_dict(), b.state_dict()
        assert list(sa) == list(sb)
        for k in sa:
            assert torch.equal(sa[k], sb[k]), k
    ranks = run_pipeline(ref, "resnet50", steps, batch)
    gold = {
        "config": {"module": "models.resnet50.gpus=4", "batch": batch, "steps": steps, "lr": 0.01, "momentum": 0.9,
                   "weight_decay": 1e-4, "seed": 0, "data_seed": 1234, "batchnorm": "training mode"},
        "description": desc,
        "losses": ranks[-1]["losses"],
        "trace": {"stage%d" % i: r["trace"] for i, r in enumerate(ranks)},
        "params": {"stage%d" % i: r["params"] for i, r in enumerate(ranks)},
        "reference_cpu_seconds": max(r["seconds"] for r in ranks),
    }
    with open(os.path.join(HERE, "resnet50_gpus4_golden.json"), "w") as f:
        json.dump(gold, f, indent=1, sort_keys=True)
    print("wrote resnet50_gpus4_golden.json; losses", gold["losses"], "in %.1f s" % gold["reference_cpu_seconds"])


# ----------------------------------------------------------------------------- GNMT (8+8 layers)
# --------------------------------------------------------------------------- #
# stage generator: the reference's generator run on two small partitioned graphs written for this purpose
# --------------------------------------------------------------------------- #
def _graph_text(nodes, edges):
    """Profile-graph text (graph/graph.py:451-461) from [(id, description, stage)] and [(src, dst)]."""
    lines = ["%s -- %s -- forward_compute_time=1.000, backward_compute_time=2.000, activation_size=4096.000, "
             "parameter_size=0.000 -- stage_id=%d" % (i, d, s) for (i, d, s) in nodes]
    lines += ["\t%s -- %s" % e for e in edges]
    return "\n".join(lines)


def stagegen_graphs():
    """Two partitioned graphs in the profiler's format: a VGG-like chain cut into three stages (the classifier's
    x.view(x.size(0), -1) straddles nothing) and a small residual network cut into three stages so that the
    first cut crosses an identity shortcut (two tensors over the boundary) and the second one a projection
    shortcut.  Node ids are deliberately not in topological order."""
    conv = "Conv2d(%d, %d, kernel_size=(3, 3), stride=(%d, %d), padding=(1, 1)%s)"
    chain = [("node1", "Input", 0),
             ("node2", conv % (3, 8, 1, 1, ""), 0), ("node3", "ReLU(inplace)", 0),
             ("node4", "MaxPool2d(kernel_size=2, stride=2, padding=0, dilation=1, ceil_mode=False)", 0),
             ("node5", conv % (8, 16, 1, 1, ""), 1), ("node6", "ReLU(inplace)", 1),
             ("node7", "MaxPool2d(kernel_size=2, stride=2, padding=0, dilation=1, ceil_mode=False)", 1),
             ("node8", "Size(0)", 1), ("node9", "View(-1)", 1),
             ("node10", "Linear(in_features=64, out_features=32, bias=True)", 1), ("node11", "ReLU(inplace)", 1),
             ("node12", "Dropout(p=0.5)", 2), ("node13", "Linear(in_features=32, out_features=10, bias=True)", 2)]
    chain_edges = [("node1", "node2"), ("node2", "node3"), ("node3", "node4"), ("node4", "node5"), ("node5", "node6"),
                   ("node6", "node7"), ("node7", "node8"), ("node7", "node9"), ("node8", "node9"), ("node9", "node10"),
                   ("node10", "node11"), ("node11", "node12"), ("node12", "node13")]
    bn = "BatchNorm2d(%d, eps=1e-05, momentum=0.1, affine=True, track_running_stats=True)"
    nb = ", bias=False"
    res = [("node1", "Input", 0),
           ("node2", conv % (3, 8, 1, 1, nb), 0), ("node3", bn % 8, 0), ("node4", "ReLU(inplace)", 0),
           # identity block: conv-bn-relu-conv-bn (+ node4) relu; the cut falls after the first ReLU of the block
           ("node21", conv % (8, 8, 1, 1, nb), 0), ("node20", bn % 8, 0), ("node19", "ReLU(inplace)", 0),
           ("node18", conv % (8, 8, 1, 1, nb), 1), ("node17", bn % 8, 1), ("node16", "Add", 1), ("node15", "ReLU(inplace)", 1),
           # projection block: main path conv(s2)-bn-relu-conv-bn, shortcut conv1x1(s2)-bn; cut inside the main path
           ("node30", conv % (8, 16, 2, 2, nb), 1), ("node31", bn % 16, 1), ("node32", "ReLU(inplace)", 1),
           ("node33", conv % (16, 16, 1, 1, nb), 2), ("node34", bn % 16, 2),
           ("node35", "Conv2d(8, 16, kernel_size=(1, 1), stride=(2, 2), bias=False)", 2), ("node36", bn % 16, 2),
           ("node37", "Add", 2), ("node38", "ReLU(inplace)", 2),
           ("node39", "AvgPool2d(kernel_size=4, stride=1, padding=0)", 2), ("node40", "Size(0)", 2), ("node41", "View(-1)", 2),
           ("node42", "Linear(in_features=16, out_features=10, bias=True)", 2)]
    res_edges = [("node1", "node2"), ("node2", "node3"), ("node3", "node4"), ("node4", "node21"), ("node21", "node20"),
                 ("node20", "node19"), ("node19", "node18"), ("node18", "node17"), ("node17", "node16"), ("node4", "node16"),
                 ("node16", "node15"), ("node15", "node30"), ("node30", "node31"), ("node31", "node32"), ("node32", "node33"),
                 ("node33", "node34"), ("node15", "node35"), ("node35", "node36"), ("node34", "node37"), ("node36", "node37"),
                 ("node37", "node38"), ("node38", "node39"), ("node39", "node40"), ("node39", "node41"), ("node40", "node41"),
                 ("node41", "node42")]
    return {"chain": ("vgg16", _graph_text(chain, chain_edges), (2, 3, 8, 8)),
            "residual": ("resnet50", _graph_text(res, res_edges), (2, 3, 8, 8))}


def stagegen_translation_graph():
    """A small translation network in the profiler's format, cut into three stages: the encoder's first layers
    (embedding, the bidirectional block, two LSTM layers with a residual connection), the rest of the encoder with the
    decoder's embedding and its attention layer (initial hidden states: a `hidden` node whose items read as None),
    and two decoder layers fed with the attention context (Concat) plus the classifier.  Hidden size 16, vocabulary
    40.  Tuple items nobody reads are left in, as the profiler leaves them."""
    H, V = 16, 40
    emu = "EmuBidirLSTM(  (bidir): LSTM(%d, %d, bidirectional=True)  (layer1): LSTM(%d, %d)  (layer2): LSTM(%d, %d))" % ((H, H) * 3)
    att = ("RecurrentAttention(  (rnn): LSTM(%d, %d)  (attn): BahdanauAttention(    (linear_q): Linear(in_features=%d, "
           "out_features=%d, bias=False)    (linear_k): Linear(in_features=%d, out_features=%d, bias=False)    (dropout): "
           "Dropout(p=0)  )  (dropout): Dropout(p=0))") % ((H, H) * 3)
    cls = "Classifier(  (classifier): Linear(in_features=%d, out_features=%d, bias=True))" % (H, V)
    drop = "Dropout(p=0.2)"
    nodes = [("node1", "Input0", 0), ("node4", "Embedding(%d, %d, padding_idx=0)" % (V, H), 0), ("node5", emu, 0),
             ("node2", "Input1", 0), ("node6", drop, 0), ("node7", "LSTM(%d, %d)" % (2 * H, H), 0),
             ("node8", "__getitem__(0)", 0), ("node9", "__getitem__(1)", 0), ("node10", drop, 0),
             ("node11", "LSTM(%d, %d)" % (H, H), 0), ("node12", "__getitem__(0)", 0), ("node13", "__getitem__(1)", 0),
             ("node14", "Add", 0),
             ("node15", drop, 1), ("node16", "LSTM(%d, %d)" % (H, H), 1), ("node17", "__getitem__(0)", 1),
             ("node18", "__getitem__(1)", 1), ("node19", "Add", 1),
             ("node3", "Input2", 1), ("node41", "Embedding(%d, %d, padding_idx=0)" % (V, H), 1), ("node40", "hidden", 1),
             ("node42", "__getitem__(0)", 1), ("node43", att, 1), ("node44", "__getitem__(0)", 1),
             ("node45", "__getitem__(1)", 1), ("node46", "__getitem__(2)", 1), ("node47", "__getitem__(3)", 1),
             ("node48", drop, 2), ("node49", "Concat(2)", 2), ("node50", "__getitem__(1)", 2),
             ("node51", "LSTM(%d, %d)" % (2 * H, H), 2), ("node52", "__getitem__(0)", 2), ("node53", "__getitem__(1)", 2),
             ("node54", drop, 2), ("node55", "Concat(2)", 2), ("node56", "__getitem__(2)", 2),
             ("node57", "LSTM(%d, %d)" % (2 * H, H), 2), ("node58", "__getitem__(0)", 2), ("node59", "__getitem__(1)", 2),
             ("node60", "Add", 2), ("node96", cls, 2)]
    edges = [("node1", "node4"), ("node4", "node5"), ("node2", "node5"), ("node5", "node6"), ("node6", "node7"),
             ("node7", "node8"), ("node7", "node9"), ("node8", "node10"), ("node10", "node11"), ("node11", "node12"),
             ("node11", "node13"), ("node12", "node14"), ("node8", "node14"), ("node14", "node15"), ("node15", "node16"),
             ("node16", "node17"), ("node16", "node18"), ("node17", "node19"), ("node14", "node19"), ("node3", "node41"),
             ("node40", "node42"), ("node41", "node43"), ("node42", "node43"), ("node19", "node43"), ("node2", "node43"),
             ("node43", "node44"), ("node43", "node45"), ("node43", "node46"), ("node43", "node47"), ("node44", "node48"),
             ("node48", "node49"), ("node46", "node49"), ("node40", "node50"), ("node49", "node51"), ("node50", "node51"),
             ("node51", "node52"), ("node51", "node53"), ("node52", "node54"), ("node54", "node55"), ("node46", "node55"),
             ("node40", "node56"), ("node55", "node57"), ("node56", "node57"), ("node57", "node58"), ("node57", "node59"),
             ("node58", "node60"), ("node52", "node60"), ("node60", "node96")]
    return "gnmt", _graph_text(nodes, edges)


def _run_reference_generator(ref, text, arch, workdir):
    """optimizer/convert_graph_to_model.py as its authors run it (a script, from its own directory), on `text`."""
    os.makedirs(workdir, exist_ok=True)
    gpath = os.path.join(workdir, "graph.txt")
    with open(gpath, "w") as f:
        f.write(text)
    out = os.path.join(workdir, "pkg")
    # graph/graph.py imports graphviz for its plots (not installed here, not used by the generator): an empty stand-in
    stubs = os.path.join(workdir, "stubs")
    os.makedirs(stubs, exist_ok=True)
    open(os.path.join(stubs, "graphviz.py"), "w").close()
    env = dict(os.environ, PYTHONPATH=stubs + os.pathsep + os.environ.get("PYTHONPATH", ""))
    subprocess.check_call([sys.executable, "convert_graph_to_model.py", "-f", gpath, "-n", "Net", "-a", arch, "-o", out],
                          cwd=os.path.join(ref, "optimizer"), stdout=subprocess.DEVNULL, env=env)
    return out


def _load_generated(pkg_dir, tag):
    """The generated package imported under a unique name; returns model(criterion) of its __init__."""
    import importlib.util
    name = "generated_%s" % tag
    spec = importlib.util.spec_from_file_location(name, os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _canonical(desc):
    """A description with every assignment of a stage's dataflow given a fresh number in order (so `a = a + b` and
    `c = a + b` read the same) and the keyword arguments of the declarations in sorted order."""
    out = {"arch": desc["arch"], "stages": []}
    for st in desc["stages"]:
        cur, flow = {}, []
        for stt in st["flow"]:
            res, op, args = stt[0], stt[1], stt[2:]
            if op == "none":                    # `x = None`: where the statement stands does not matter
                cur[res] = "None"
                continue
            args = [cur[a] if isinstance(a, str) else a for a in args]
            cur[res] = "v%d" % len(flow)
            flow.append([cur[res], op] + args)
        out["stages"].append({"modules": [[n, k, dict(sorted(kw.items()))] for n, k, kw in st["modules"]], "flow": flow,
                              "returns": [cur[r] for r in st["returns"]],
                              "inputs": list(st["inputs"]), "outputs": list(st["outputs"])})
    return out


def make_stagegen(ref):
    import hashlib
    import tempfile
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from pipedream_b200 import stagegen, stages as pd_stages
    golden = {"graphs": {}, "checked_on_reference_graphs": {}}
    work = tempfile.mkdtemp(prefix="pd_stagegen_")

    def generated_description(text, arch, tag):
        pkg = _run_reference_generator(ref, text, arch, os.path.join(work, tag))
        mod = _load_generated(pkg, tag)
        torch.manual_seed(0)
        model = mod.model(torch.nn.CrossEntropyLoss())
        desc = {"arch": mod.arch(), "stages": []}
        for (m, ins, outs) in model[:-1]:
            d = describe_stage(m)
            d["inputs"], d["outputs"] = list(ins), list(outs)
            desc["stages"].append(d)
        return desc, model

    for name, (arch, text, shape) in stagegen_graphs().items():
        desc, model = generated_description(text, arch, name)
        mine = stagegen.describe(text, arch)
        assert _canonical(mine) == _canonical(desc), name
        # the generated stages run on a seeded input; the description built here must give the same numbers
        torch.manual_seed(1)
        x = torch.randn(*shape)
        vals = {"input0": x}
        for (m, ins, outs) in model[:-1]:
            m.eval()
            r = m(*[vals[i] for i in ins])
            r = r if isinstance(r, tuple) else (r,)
            vals.update(dict(zip(outs, r)))
        last = model[-2][2][0]
        sd = {}
        for si, (m, _, _) in enumerate(model[:-1]):
            for k, v in m.state_dict().items():
                sd["%d.%s" % (si, k)] = tensor_checksum(v)
        golden["graphs"][name] = {"arch": arch, "text": text, "input_shape": list(shape), "description": desc,
                                  "output": vals[last].detach().double().flatten().tolist(), "state_dict": sd}
    # the translation model's node kinds: descriptions compared here and in the test, numbers in the test only on
    # shapes (the composite blocks initialise themselves, in an order of their own)
    _import_reference(ref, domain="translation")
    _inject_pack_utils()
    arch, text = stagegen_translation_graph()
    desc, model = generated_description(text, arch, "translation")
    mine = stagegen.describe(text, arch)
    assert _canonical(mine) == _canonical(desc), "translation"
    shapes = {}
    for si, (m, _, _) in enumerate(model[:-1]):
        for k, v in m.state_dict().items():
            shapes["%d.%s" % (si, k)] = list(v.shape)
    golden["graphs"]["translation"] = {"arch": arch, "text": text, "description": desc, "state_dict_shapes": shapes}
    # the reference's profile of its large translation model, cut here into four stages at node numbers (the
    # partitioned file the shipped stages were generated from is not in the tree)
    gpath = os.path.join(ref, "profiler", "translation", "profiles", "gnmt_large", "graph.txt")
    gtext = open(gpath).read()

    def cut(nid):
        n = int(nid[4:])
        if n in (1, 2):
            return 0
        if n == 3:
            return 1
        return 0 if n <= 23 else (1 if n <= 47 else (2 if n <= 74 else 3))
    glines = gtext.strip().split("\n")
    ptext = "\n".join([ln + " -- stage_id=%d" % cut(ln.split(" -- ")[0]) for ln in glines if not ln.startswith("\t")] +
                      [ln for ln in glines if ln.startswith("\t")])
    desc, _ = generated_description(ptext, "gnmt_large", "gnmt_large_cut")
    same = _canonical(stagegen.describe(ptext, "gnmt_large")) == _canonical(desc)
    assert same, "gnmt_large"
    golden["checked_on_reference_graphs"]["profiles/gnmt_large/graph.txt, cut into 4 stages"] = {
        "sha256": hashlib.sha256(gtext.encode()).hexdigest(), "stages": len(desc["stages"]),
        "modules": sum(len(st["modules"]) for st in desc["stages"]), "equal_to_generator_output": same}
    # the same profile partitioned by this repository's planner for 4 GPUs (reference cost model): the generator and
    # the front end must agree on whatever cut comes out
    from pipedream_b200 import partition
    _, plan4, planned = partition.plan_graph(stagegen.Graph.parse(gtext), 4, 16e9, straight=True, cost="reference")
    desc, _ = generated_description(planned, "gnmt_large", "gnmt_large_planned")
    same = _canonical(stagegen.describe(planned, "gnmt_large")) == _canonical(desc)
    assert same, "gnmt_large planned"
    golden["checked_on_reference_graphs"]["profiles/gnmt_large/graph.txt, partitioned by partition.plan_graph for 4 GPUs"] = {
        "sha256": hashlib.sha256(gtext.encode()).hexdigest(), "stages": len(desc["stages"]),
        "layers_per_stage": [e - b for b, e, _ in plan4], "equal_to_generator_output": same}
    # the reference's own partitioned test graphs: checked here, where the reference is at hand; only the outcome,
    # the stage count and the file's digest are recorded
    for fname, arch in (("vgg16_partitioned.txt", "vgg16"), ("resnet50_partitioned.txt", "resnet50")):
        path = os.path.join(ref, "graph", "test_graphs", fname)
        text = open(path).read()
        desc, _ = generated_description(text, arch, fname.split(".")[0])
        mine = stagegen.describe(text, arch)
        same = _canonical(mine) == _canonical(desc)
        assert same, fname
        golden["checked_on_reference_graphs"][fname] = {
            "sha256": hashlib.sha256(text.encode()).hexdigest(), "stages": len(desc["stages"]),
            "modules": sum(len(s["modules"]) for s in desc["stages"]), "equal_to_generator_output": same}
    with open(os.path.join(HERE, "stagegen_golden.json"), "w") as f:
        json.dump(golden, f, indent=1)
    print("wrote stagegen_golden.json", golden["checked_on_reference_graphs"])


def _inject_pack_utils():
    """Pure-torch stand-in for the reference's pack_utils CUDA extension (csrc/pack_utils_kernel.cu:24-63,
    pack_utils.cpp:13-31), which does not build against current PyTorch."""
    import types
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from pipedream_b200.gnmt_blocks import _revert_varlen_torch
    stub, c = types.ModuleType("pack_utils"), types.ModuleType("pack_utils._C")
    c.revert_varlen_tensor = lambda x, lengths: _revert_varlen_torch(x, lengths)

    def set_mask_cpp(lengths):
        T = int(lengths[0])
        return (torch.arange(T).unsqueeze(1) < lengths.unsqueeze(0)).to(torch.uint8)
    c.set_mask_cpp = set_mask_cpp
    stub._C = c
    sys.modules["pack_utils"], sys.modules["pack_utils._C"] = stub, c


GNMT_PIPE = {"batch": 8, "min_len": 6, "max_len": 14, "lr": 2e-3, "weight_decay": 1e-4, "data_seed": 4321}


def gnmt_worker(ref, rank, steps, out_path):
    """One rank of the reference's 4-stage GNMT pipeline (models.gnmt_large.gpus=4, one stage per rank) through the
    reference runtime in its translation mode: variable-length batches sorted by source length, LabelSmoothing,
    AdamWithWeightStashing with 4, 3, 2, 1 weight versions from the first to the last stage."""
    _shim_cpu()
    _import_reference(ref, "translation")
    _inject_pack_utils()
    import runtime as ref_runtime
    import adam as ref_adam
    import communication as ref_comm
    _shim_transport(ref_comm)
    from seq2seq.train.smoothing import LabelSmoothing
    from pipedream_b200.stages import SyntheticTranslation
    cfg = GNMT_PIPE
    torch.manual_seed(0)
    module = importlib.import_module("models.gnmt_large.gpus=4")
    model = module.model(LabelSmoothing(0, 0.1))
    for (m, _, _) in model[:-1]:
        for sub in m.modules():
            if isinstance(sub, torch.nn.Dropout):
                sub.p = 0.0
    B, T = cfg["batch"], cfg["max_len"]
    shapes = {"input0": [T, B], "input1": [B], "input2": [T, B], "target": [T * B], "target_length": [B]}
    dtypes = {"input0": torch.int64, "input1": torch.int64, "input2": torch.int64, "target": torch.int64,
              "target_length": torch.int32}
    dests = {"input0": 0, "input1": 0, "input2": 0}
    for module_id, (stage, inputs, outputs) in enumerate(model[:-1]):        # translation/main_with_runtime.py:161-184
        ins = []
        for name in inputs:
            if name in dests:
                dests[name] = module_id
            ins.append(torch.ones(tuple(shapes[name]), dtype=dtypes[name]))
        with torch.no_grad():
            o = stage(*ins)
        o = o if isinstance(o, tuple) else (o,)
        for name, t in zip(outputs, o):
            shapes[name] = list(t.size())
            dtypes[name] = t.dtype
    shapes = {k: tuple(v) for k, v in shapes.items()}
    conf = {"module_to_stage_map": [0, 1, 2, 3, 3], "stage_to_rank_map": {s: [s] for s in range(4)}, "stage_to_depth_map": None}
    r = ref_runtime.StageRuntime(
        model=model, distributed_backend="gloo", fp16=False, loss_scale=1, training_tensor_shapes=shapes,
        eval_tensor_shapes=dict(shapes), training_tensor_dtypes=dtypes, inputs_module_destinations=dests,
        target_tensor_names={"target", "target_length"}, configuration_maps=conf, master_addr="127.0.0.1",
        rank=rank, local_rank=rank, num_ranks_in_server=1, verbose_freq=0, model_type=ref_runtime.TRANSLATION)
    opt = ref_adam.AdamWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1,
                                          num_versions=r.num_warmup_minibatches + 1, lr=cfg["lr"],
                                          weight_decay=cfg["weight_decay"])
    n = steps
    r.train(n)
    r.set_loader(SyntheticTranslation(B, n, seed=cfg["data_seed"], min_len=cfg["min_len"], max_len=cfg["max_len"])
                 if r.stage == 0 else None)
    losses, trace = [], []

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
            losses.append([float(r.tensors[-1]["loss"]), float(r.loss)])
        bwd(i)
    for i in range(w):
        bwd(n - w + i)
    r.wait()
    params = {}
    for mi, m in enumerate(r.modules()):
        for k, v in m.state_dict().items():
            if v is not None:
                params["module%d.%s" % (mi, k)] = tensor_checksum(v)
    with open(out_path, "w") as f:
        json.dump({"rank": rank, "stage": r.stage, "num_versions": opt.num_versions, "losses": losses, "trace": trace,
                   "params": params, "shapes": {k: list(v) for k, v in shapes.items()},
                   "dtypes": {k: str(v) for k, v in dtypes.items()}, "inputs_module_destinations": dests}, f)


def make_gnmt_pipeline(ref, steps=20):
    import time
    t0 = time.time()
    procs, outs = [], []
    for rank in range(4):
        out_path = "/tmp/gnmt_pipe_rank%d.json" % rank
        outs.append(out_path)
        env = dict(os.environ, OMP_NUM_THREADS=str(max(1, (os.cpu_count() or 4) // 4)), PYTHONDONTWRITEBYTECODE="1")
        procs.append(subprocess.Popen([sys.executable, "-O", os.path.abspath(__file__), "--ref", ref, "--worker", str(rank),
                                       "--steps", str(steps), "--out", out_path, "--pipeline", "gnmt"], env=env))
    _wait_all(procs, 1500)
    ranks = [json.load(open(o)) for o in outs]
    gold = {"config": dict(GNMT_PIPE, module="models.gnmt_large.gpus=4", steps=steps, seed=0, smoothing=0.1,
                           optimizer="Adam", dropout="disabled (p=0)", num_versions=[r["num_versions"] for r in ranks],
                           inputs_module_destinations=ranks[0]["inputs_module_destinations"]),
            "losses": [x[0] for x in ranks[3]["losses"]], "losses_per_token": [x[1] for x in ranks[3]["losses"]],
            "trace": {"stage%d" % i: r["trace"] for i, r in enumerate(ranks)},
            "params": {"stage%d" % i: r["params"] for i, r in enumerate(ranks)},
            "shapes": ranks[0]["shapes"], "dtypes": ranks[0]["dtypes"], "reference_cpu_seconds": time.time() - t0}
    with open(os.path.join(HERE, "gnmt_pipeline_golden.json"), "w") as f:
        json.dump(gold, f, indent=1, sort_keys=True)
    print("wrote gnmt_pipeline_golden.json; losses", [round(x, 3) for x in gold["losses"]], "in %.1f s" % gold["reference_cpu_seconds"])


def make_gnmt(ref, steps=3, batch=8):
    """The reference's gnmt_large stage modules (4 stages run back to back in one process), its
    LabelSmoothing criterion and AdamWithWeightStashing, on CPU.  The reference's pack_utils CUDA
    extension does not build against current PyTorch; a pure-torch stand-in with the semantics of
    csrc/pack_utils_kernel.cu:24-63 and pack_utils.cpp:13-31 is injected in its place."""
    _shim_cpu()
    _import_reference(ref, "translation")
    _inject_pack_utils()
    from pipedream_b200.stages import SyntheticTranslation
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
    ap.add_argument("--pipeline", default="vgg16")
    ap.add_argument("--f64", action="store_true")
    a = ap.parse_args()
    if a.worker is not None and a.pipeline == "gnmt":
        gnmt_worker(a.ref, a.worker, a.steps, a.out)
    elif a.worker is not None:
        vgg16_worker(a.ref, a.worker, a.steps, a.batch, a.out, a.pipeline, a.f64)
    else:
        if a.only in (None, "routing"):
            subprocess.check_call([sys.executable, "-O", "-c",
                                   "import sys; sys.path.insert(0, %r); import make_golden; make_golden.make_routing(%r)" % (HERE, a.ref)])
        if a.only in (None, "partition"):
            subprocess.check_call([sys.executable, "-O", "-c",
                                   "import sys; sys.path.insert(0, %r); import make_golden; make_golden.make_partition(%r)" % (HERE, a.ref)])
        if a.only in (None, "signatures"):
            subprocess.check_call([sys.executable, "-O", "-c",
                                   "import sys; sys.path.insert(0, %r); import make_golden; make_golden.make_signatures(%r)" % (HERE, a.ref)])
        if a.only in (None, "stagegen"):
            subprocess.check_call([sys.executable, "-c",
                                   "import sys; sys.path.insert(0, %r); import make_golden; make_golden.make_stagegen(%r)" % (HERE, a.ref)])
        if a.only in (None, "stashing"):
            subprocess.check_call([sys.executable, "-O", "-c",
                                   "import sys; sys.path.insert(0, %r); import make_golden; make_golden.make_stashing(%r)" % (HERE, a.ref)])
        if a.only in (None, "vgg16"):
            make_vgg16(a.ref, a.steps, a.batch)
        if a.only in (None, "vgg16_f64"):
            make_vgg16(a.ref, a.steps, a.batch, f64=True)
        if a.only in (None, "resnet50"):
            subprocess.check_call([sys.executable, "-O", "-c",
                                   "import sys; sys.path.insert(0, %r); import make_golden; make_golden.make_resnet50(%r)" % (HERE, a.ref)])
        if a.only in (None, "gnmt_pipeline"):
            make_gnmt_pipeline(a.ref, a.steps)
        if a.only in (None, "gnmt"):
            subprocess.check_call([sys.executable, "-O", "-c",
                                   "import sys; sys.path.insert(0, %r); import make_golden; make_golden.make_gnmt(%r)" % (HERE, a.ref)])
