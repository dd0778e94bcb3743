"""Multi-GPU arm of bench.py: one process per GPU (torch.distributed.run), VGG-16 bf16.

Partitions (stage:replicas), per-replica batch 64 in stage 0, chosen the way the reference's
partitioner splits VGG-16 - convolutions replicated, the parameter-heavy Linear layers on
one GPU - once there are enough GPUs for it:

    N = 2 : 1 stage x 2 replicas (data parallel; dp_conf.json form)
    N = 4 : stage 0 (conv1_1 .. pool5 + flatten) x 3, stage 1 (FC6-8) x 1   (hybrid 3:1)
    N = 8 : stage 0 x 7, stage 1 x 1                                        (hybrid 7:1)

Boundary tensors move over the NVLink peer channels; the replicas of a stage sum their flat
gradient arena with one NCCL all-reduce per step.  Every rank times its own K steady-state
steps with CUDA events between barriers; the job time is the maximum over ranks.
"""
import os

import torch
import torch.distributed as dist

from bench import BATCH, METRIC, UNIT, ClockSampler, CyclingLoader, peaks, FLOPS_PER_SAMPLE


def partition_for(n):
    if n == 2:
        return "gpus=1", {"module_to_stage_map": [0, 0], "stage_to_rank_map": {0: [0, 1]}, "stage_to_depth_map": None}, "dp2"
    if n >= 3:
        return "gpus=16", {"module_to_stage_map": [0, 1, 1],
                           "stage_to_rank_map": {0: list(range(n - 1)), 1: [n - 1]},
                           "stage_to_depth_map": None}, "hybrid %d:1" % (n - 1)
    raise ValueError(n)


def build_worker(pkg_name, conf, rank, local_rank, fp16=True):
    from pipedream_b200 import runtime, sgd, stages
    torch.manual_seed(0)
    pkg = stages.vgg16(pkg_name)
    model = pkg.model(torch.nn.CrossEntropyLoss())
    act = torch.bfloat16 if fp16 else torch.float32
    shapes = {"input0": (BATCH, 3, 224, 224), "target": (BATCH,)}
    dtypes = {"input0": torch.int64, "target": torch.int64}
    if pkg_name == "gpus=16":
        shapes.update({"out0": (BATCH, 25088), "out1": (BATCH, 1000)})
    else:
        shapes.update({"out0": (BATCH, 1000)})
    for k in shapes:
        if k.startswith("out"):
            dtypes[k] = act
    r = runtime.StageRuntime(
        model=model, distributed_backend="p2p", fp16=fp16, loss_scale=1, training_tensor_shapes=shapes,
        eval_tensor_shapes=dict(shapes), training_tensor_dtypes=dtypes, inputs_module_destinations={"input": 0},
        target_tensor_names={"target"}, configuration_maps=conf,
        master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1"), rank=rank, local_rank=local_rank,
        num_ranks_in_server=1, verbose_freq=0, model_type=runtime.IMAGE_CLASSIFICATION)
    opt = sgd.SGDWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1,
                                    num_versions=r.num_warmup_minibatches + 1,
                                    lr=r.get_adjusted_learning_rate(0.01), momentum=0.9, weight_decay=5e-4)
    return r, opt


RESNET_BATCH = 128
RESNET_FLOPS_PER_SAMPLE = 24.30e9


def build_resnet_worker(n, rank, local_rank, fp16=True):
    """ResNet-50 as an n-stage straight pipeline (one stage per GPU), batch 128, SGD 0.1 / 0.9 / 1e-4."""
    from pipedream_b200 import runtime, sgd, stages
    torch.manual_seed(0)
    pkg = stages.resnet50(n)
    model = pkg.model(torch.nn.CrossEntropyLoss())
    act = torch.bfloat16 if fp16 else torch.float32
    shapes = pkg.boundary_shapes(RESNET_BATCH)
    dtypes = {k: (act if k.startswith("out") else torch.int64) for k in shapes}
    conf = dict(pkg.conf, stage_to_depth_map=None)
    r = runtime.StageRuntime(
        model=model, distributed_backend="p2p", fp16=fp16, loss_scale=1, training_tensor_shapes=shapes,
        eval_tensor_shapes=dict(shapes), training_tensor_dtypes=dtypes, inputs_module_destinations={"input": 0},
        target_tensor_names={"target"}, configuration_maps=conf,
        master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1"), rank=rank, local_rank=local_rank,
        num_ranks_in_server=1, verbose_freq=0, model_type=runtime.IMAGE_CLASSIFICATION)
    opt = sgd.SGDWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1,
                                    num_versions=r.num_warmup_minibatches + 1, lr=0.1, momentum=0.9, weight_decay=1e-4)
    return r, opt, conf


# --------------------------------------------------------------------------- #
# evidence that what crosses NVLink arrives intact, and that replicas average what they computed
# --------------------------------------------------------------------------- #
def _checksum(t):
    d = t.detach().double()
    return [d.sum().item(), d.abs().sum().item(), int(d.numel())]


def parity_probe(r, opt, loader):
    """One extra minibatch per stage-0 replica with instruments on: every floating tensor a rank pushes into a
    peer channel and every one it takes out is summed in fp64 on both ends, and the flat gradient arena of a
    replicated stage is summed before and after the all-reduce.  Rank 0 gathers the records: each sent checksum
    must appear, bit for bit, among the received ones, and every replica's arena after the all-reduce must be the
    sum of the replicas' arenas before it (recomputed from the gathered partial sums)."""
    from pipedream_b200 import schedule
    rec = {"rank": r.rank, "stage": r.stage, "sent": [], "received": [], "grad_before": None, "grad_after": None}
    h = r.comm_handler
    orig_send, orig_recv = h.send, h.recv

    def send(name, tensor, forward_minibatch_id, backward_minibatch_id, backward=False):
        if tensor.is_floating_point():
            rec["sent"].append([name, int(backward)] + _checksum(tensor))
        return orig_send(name, tensor, forward_minibatch_id, backward_minibatch_id, backward=backward)

    def recv(name, forward_minibatch_id, backward_minibatch_id, backward=False):
        t = orig_recv(name, forward_minibatch_id, backward_minibatch_id, backward=backward)
        if t.is_floating_point():
            rec["received"].append([name, int(backward)] + _checksum(t))
        return t

    h.send, h.recv = send, recv
    orig_sync = opt._grad_sync
    if orig_sync is not None:
        def sync(arena):
            rec["grad_before"] = _checksum(arena)
            out = orig_sync(arena)
            rec["grad_after"] = _checksum(arena)
            return out
        opt._grad_sync = sync
    scale = r.num_ranks_in_first_stage / r.num_ranks_in_stage if r.stage else 1
    n = int(round(1 * scale))
    r.train(n)
    r.set_loader(loader if r.stage in (0, None) else None)
    schedule.train_1f1b(r, opt, n)
    torch.cuda.synchronize()
    h.send, h.recv = orig_send, orig_recv
    opt._grad_sync = orig_sync
    allrec = [None] * dist.get_world_size()
    dist.all_gather_object(allrec, rec)
    if r.rank != 0:
        return None
    sent = sorted(tuple(x) for a in allrec for x in a["sent"])
    got = sorted(tuple(x) for a in allrec for x in a["received"])
    out = {"boundary_tensors_sent": len(sent), "boundary_tensors_received": len(got), "boundary_match": sent == got}
    stages = {}
    for a in allrec:
        if a["grad_before"] is not None:
            stages.setdefault(a["stage"], []).append(a)
    ok, worst = True, 0.0
    for st, members in stages.items():
        want = sum(m["grad_before"][0] for m in members)
        scale_ = max(sum(m["grad_before"][1] for m in members), 1e-30)
        for m in members:
            err = abs(m["grad_after"][0] - want) / scale_
            worst = max(worst, err)
            ok = ok and err <= 1e-5
    out["allreduce_replicas"] = {str(k): len(v) for k, v in stages.items()}
    out["allreduce_sum_rel_err"] = worst
    out["allreduce_match"] = ok
    return out


def nvlink_peer_copy_gbs(nbytes=1 << 30):
    """Measured once on rank 0: device-to-device copy cuda:0 -> cuda:1 with the copy engine (GB/s)."""
    if torch.cuda.device_count() < 2 or not torch.cuda.can_device_access_peer(0, 1):
        return None
    a = torch.empty(nbytes, dtype=torch.uint8, device="cuda:0")
    b = torch.empty(nbytes, dtype=torch.uint8, device="cuda:1")
    for _ in range(2):
        b.copy_(a)
    torch.cuda.synchronize(0); torch.cuda.synchronize(1)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.device(0):
        s.record()
        for _ in range(5):
            b.copy_(a)
        e.record()
    torch.cuda.synchronize(0); torch.cuda.synchronize(1)
    ms = s.elapsed_time(e) / 5
    del a, b
    return round(nbytes / (ms * 1e-3) / 1e9, 1)


# Per-sample work of the VGG-16 stages (2 flops per multiply-add, counted on the reference modules; elements in /
# out of contractions and out of the other leaves) - the numbers the stage roofline below is built from.
VGG_STAGE_WORK = {
    "gpus=1": [{"gflop": 92.65, "elems": (9.11e6, 13.56e6, 15.10e6), "params": 138.36e6}],
    "gpus=16": [{"gflop": 91.90, "elems": (9.08e6, 13.55e6, 15.08e6), "params": 14.71e6},
                {"gflop": 0.74, "elems": (33e3, 9e3, 16e3), "params": 123.64e6}],
}


def stage_roofline(pkg_name, conf, batch, ms_per_step, nvlink_gbs, boundary_bytes):
    """t_s = max(F_s / P_tensor, Q_s / BW_hbm) + X_s / BW_nvlink per stage and minibatch, and how much of the measured
    minibatch period of that stage it explains.  Q_s is a minimal-traffic model: every contraction reads its input and
    writes its output once forward, reads the output gradient and the saved input and writes the input gradient
    backward; every other leaf reads and writes its tensor once per pass; weights are read three times and the
    fused optimizer moves 22 bytes per parameter."""
    pk = peaks()
    out = []
    r0 = len(conf["stage_to_rank_map"][0])
    for s, w in enumerate(VGG_STAGE_WORK[pkg_name]):
        rs = len(conf["stage_to_rank_map"][s]) if s in conf["stage_to_rank_map"] else 1
        cin, cout, other = w["elems"]
        q = 2.0 * batch * (3 * cin + 2 * cout + 4 * other) + w["params"] * (3 * 2 + 22)
        f = w["gflop"] * 1e9 * batch
        x = boundary_bytes * 2 if len(VGG_STAGE_WORK[pkg_name]) > 1 else 0      # activations one way, gradients the other
        t = max(f / (pk["bf16_tflops_sustained"] * 1e12), q / (pk["hbm_gbs"] * 1e9)) + (x / (nvlink_gbs * 1e9) if nvlink_gbs else 0.0)
        period = ms_per_step * 1e-3 * rs / r0          # measured time per minibatch of one replica of this stage
        out.append({"stage": s, "replicas": rs, "tflop_per_minibatch": round(f / 1e12, 3), "hbm_gb_per_minibatch": round(q / 1e9, 3),
                    "nvlink_mb_per_minibatch": round(x / 1e6, 2), "roofline_ms": round(t * 1e3, 3),
                    "measured_ms": round(period * 1e3, 3), "frac": round(t / period, 4),
                    "bound": "tensor" if f / (pk["bf16_tflops_sustained"] * 1e12) >= q / (pk["hbm_gbs"] * 1e9) else "hbm"})
    return out


def _backward(r, opt):
    opt.zero_grad()
    opt.load_old_params()
    r.run_backward()
    opt.load_new_params()
    opt.step()


def run_phase(r, opt, loader, n0, warm0, read_loss):
    """One 'epoch' of n0 + warm0 minibatches per stage-0 replica.  The first warm0 (scaled to this
    stage) steady-state iterations are untimed; returns the milliseconds of the rest on this rank."""
    scale = r.num_ranks_in_first_stage / r.num_ranks_in_stage if r.stage else 1
    n = int(round((n0 + warm0) * scale))
    skip = int(round(warm0 * scale))
    r.train(n)
    r.set_loader(loader if r.stage in (0, None) else None)
    w = r.num_warmup_minibatches
    for _ in range(w):
        r.run_forward()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = []
    for i in range(n - w):
        if i == skip:
            torch.cuda.synchronize()
            dist.barrier()
            start.record()
        if len(marks) >= 2:
            marks.pop(0).synchronize()      # bounded run-ahead of the host (see bench_gnmt.run)
        r.run_forward()
        if read_loss and r.is_criterion:
            r.loss.item()
        _backward(r, opt)
        ev = torch.cuda.Event()
        ev.record()
        marks.append(ev)
    for _ in range(w):
        _backward(r, opt)
    end.record()
    torch.cuda.synchronize()
    r.wait()
    dist.barrier()
    return start.elapsed_time(end)


def run_gpu_multi(gpus, steps, warmup, model="vgg16"):
    from pipedream_b200 import _lib
    from pipedream_b200 import functional as pf
    rank = int(os.environ["RANK"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    world = int(os.environ["WORLD_SIZE"])
    assert world == gpus, "launch with torch.distributed.run --nproc-per-node %d" % gpus
    torch.cuda.set_device(local_rank)
    if model == "resnet50":
        pkg_name, label, batch, flops = "resnet50", "%d-stage straight pipeline" % world, RESNET_BATCH, RESNET_FLOPS_PER_SAMPLE
        r, opt, conf = build_resnet_worker(world, rank, local_rank)
    else:
        pkg_name, conf, label = partition_for(world)
        batch, flops = BATCH, FLOPS_PER_SAMPLE
        r, opt = build_worker(pkg_name, conf, rank, local_rank)
    first = r.stage in (0, None)
    parity = parity_probe(r, opt, CyclingLoader(batch, "cuda", pool=1, seed=77 + rank) if first else None)
    nvl = nvlink_peer_copy_gbs() if rank == 0 else None
    dist.barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    _lib.count_calls(True)
    ms = run_phase(r, opt, CyclingLoader(batch, "cuda", seed=1234 + 1000 * rank) if first else None, steps, warmup, False)
    launches = _lib.launches_counted()
    _lib.count_calls(False)
    clocks = sampler.stop() if sampler else None
    host = CyclingLoader(batch, "pinned", seed=1234 + 1000 * rank) if first else None
    ms_e2e = run_phase(r, opt, host, steps, max(1, warmup // 2), True)
    if pf.gemm_poll_error() != 0:
        raise RuntimeError("a tcgen05 kernel reported a bounded wait that ran out")
    t = torch.tensor([ms, ms_e2e, float(launches)], dtype=torch.float64, device="cuda")
    tmax = t.clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    r0 = len(conf["stage_to_rank_map"][0])
    samples = batch * r0 * steps
    secondary = None
    if model == "vgg16" and world in (2, 4, 8) and os.environ.get("PD_BENCH_NO_SECONDARY") != "1":
        # the other network of the headline metric on the same GPUs (N = 8: four stages x two replicas)
        import gc
        import bench_gnmt
        del r, opt
        gc.collect()
        torch.cuda.empty_cache()
        try:
            g = bench_gnmt.run_multi(world, min(steps, 30), warmup)
            if g is not None:
                secondary = {"gnmt": {k: g[k] for k in ("metric", "value", "unit", "steps", "ms_per_step", "e2e", "gpu_launches",
                                                              "stage_roofline")}}
                secondary["gnmt"]["config"] = g["config"]
        except Exception as e:
            secondary = {"gnmt": {"error": "%s: %s" % (type(e).__name__, e)}}
    if rank != 0:
        return None
    pk = peaks()
    ms_job, ms_job_e2e = tmax[0].item(), tmax[1].item()
    value = samples / (ms_job * 1e-3)
    return {
        "metric": METRIC if model == "vgg16" else "resnet50_train_samples_per_sec", "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_job / steps, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": ("VGG-16 bf16 training, batch 64 per stage-0 replica of 3x224x224 N(0,1) images, SGD "
                                "momentum 0.9, 1F1B with weight stashing") if model == "vgg16" else
                               ("ResNet-50 bf16 training (BN in training mode), batch 128 of 3x224x224 N(0,1) images, SGD "
                                "momentum 0.9 lr 0.1 wd 1e-4, 1F1B with weight stashing (depth = stage count at stage 0)"),
                   "global_batch": batch * r0,
                   "parallelism": label, "l2": "no flush: per-step activations (>1 GB) exceed the 126 MB L2"},
        "clocks": clocks,
        "e2e": {"value": round(samples / (ms_job_e2e * 1e-3), 2), "unit": UNIT,
                "h2d_bytes_per_step": (batch * 3 * 224 * 224 * 4 + batch * 8) * r0, "d2h_bytes_per_step": 4 * (r0 if pkg_name == "gpus=1" else 1),
                "ms_per_step": round(ms_job_e2e / steps, 3)},
        "gpu_launches": int(t[2].item()),
        "parity": parity,
        "nvlink_peer_copy_gbs": nvl,
        "stage_roofline": stage_roofline(pkg_name, conf, batch, tmax[0].item() / steps, nvl,
                                         batch * 25088 * 2) if model == "vgg16" else None,
        "secondary": secondary,
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel", "achieved": round(flops * value / 1e12 / world, 1),
                     "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": round(flops * value / 1e12 / world / pk["bf16_tflops_sustained"], 4),
                     "traffic": None, "note": "whole-step algorithmic FLOP rate per GPU (model FLOPs / job time / GPUs); "
                                              "the per-kernel figure is reported by the 1-GPU run"},
    }
