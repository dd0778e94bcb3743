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
import time

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
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel", "achieved": round(flops * value / 1e12 / world, 1),
                     "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": round(flops * value / 1e12 / world / pk["bf16_tflops_sustained"], 4),
                     "traffic": None, "note": "whole-step algorithmic FLOP rate per GPU (model FLOPs / job time / GPUs); "
                                              "the per-kernel figure is reported by the 1-GPU run"},
    }
