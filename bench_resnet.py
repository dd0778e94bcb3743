"""ResNet-50 arm of bench.py (`python bench.py --model resnet50`): the whole network (bottleneck blocks,
BatchNorm in training mode) as one stage on one GPU, bf16, batch 64 of 3x224x224 images, SGD momentum
0.9 lr 0.1 wd 1e-4 - the optimizer settings of the reference's driver script for this network."""
import os
import time

import torch

from bench import ClockSampler, CyclingLoader, one_step, peaks, timed_loop

BATCH = 64
METRIC = "resnet50_train_samples_per_sec"
FLOPS_PER_SAMPLE = 24.30e9       # 8.18 forward + 16.12 backward, 2 flops per multiply-add


def build(fp16=True):
    from pipedream_b200 import runtime, sgd, stages
    torch.manual_seed(0)
    model = stages.resnet50(1).model(torch.nn.CrossEntropyLoss())
    r = runtime.StageRuntime(
        model=model, distributed_backend=None, fp16=fp16, loss_scale=1, training_tensor_shapes={},
        eval_tensor_shapes={}, training_tensor_dtypes={}, inputs_module_destinations={"input": 0},
        target_tensor_names={"target"},
        configuration_maps={"module_to_stage_map": None, "stage_to_rank_map": None, "stage_to_depth_map": None},
        master_addr=None, rank=None, local_rank=0, num_ranks_in_server=1, verbose_freq=0,
        model_type=runtime.IMAGE_CLASSIFICATION)
    opt = sgd.SGDWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1, num_versions=1, lr=0.1,
                                    momentum=0.9, weight_decay=1e-4)
    return r, opt


def cpu_baseline(batch=16):
    """The same network from plain torch modules, trained by the CPU oracle: one minibatch of `batch`."""
    from oracle import pipedream_oracle as oracle
    from pipedream_b200 import stages
    torch.manual_seed(0)
    st = stages.resnet50(1).stages()[0]
    model = [(st, ["input0"], ["out0"]), (torch.nn.CrossEntropyLoss(), ["out0"], ["loss"])]
    pipe = oracle.PipelineOracle(model, [0, 0], {0: [0]}, None, "SGD", dict(lr=0.1, momentum=0.9, weight_decay=1e-4))
    pipe.run({0: stages.SyntheticImages(batch, 1)}, 1)
    t0 = time.time()
    pipe.run({0: stages.SyntheticImages(batch, 2, seed=99)}, 2)
    dt = time.time() - t0
    return {"value": 2 * batch / dt, "unit": "samples/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": "2 minibatches of %d images, fp32, after 1 untimed minibatch" % batch}


def run(steps, warmup, with_cpu):
    from pipedream_b200 import _lib
    from pipedream_b200 import functional as pf
    torch.cuda.set_device(0)
    r, opt = build()
    r.train(2 * (steps + warmup) + 8)
    r.set_loader(CyclingLoader(BATCH, "cuda"))
    sampler = ClockSampler(0)
    sampler.start()
    for _ in range(warmup):
        one_step(r, opt, False)
    torch.cuda.synchronize()
    _lib.count_calls(True)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        one_step(r, opt, False)
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e)
    launches, calls = _lib.launches_counted(), dict(_lib.COUNTERS)
    _lib.count_calls(False)
    clocks = sampler.stop()
    # instrumented pass (CUDA events around every contraction), outside every throughput figure
    isteps = 2
    pf.timeline = pf.ContractionTimeline()
    for _ in range(isteps):
        one_step(r, opt, False)
    torch.cuda.synchronize()
    tl = pf.timeline.summary()
    if os.environ.get("PD_BENCH_DETAIL"):
        with open(os.environ["PD_BENCH_DETAIL"], "w") as f:
            for k, v in sorted(pf.timeline.per_shape().items()):
                f.write("%-44s launches/step %3d  ms/step %7.3f  TFLOP/s %7.1f\n" % (
                    k, v[0] // isteps, v[2] / isteps, v[1] / max(v[2], 1e-9) / 1e9))
    pf.timeline = None
    host = CyclingLoader(BATCH, "pinned")
    r.set_loader(host)
    ms_e2e = timed_loop(r, opt, steps, 2, True)
    if pf.gemm_poll_error() != 0:
        raise RuntimeError("a tcgen05 kernel reported a bounded wait that ran out")
    pk = peaks()
    flops = sum(v[1] for v in tl.values())
    kms = sum(v[2] for v in tl.values())
    ach = flops / (kms * 1e-3) / 1e12 if kms > 0 else 0.0
    out = {
        "metric": METRIC, "value": round(BATCH * steps / (ms * 1e-3), 2), "unit": "samples/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "ResNet-50 bf16 training step (BatchNorm in training mode), batch 64 of 3x224x224 "
                               "N(0,1) images, SGD momentum 0.9 lr 0.1 wd 1e-4, one stage on one GPU",
                   "global_batch": BATCH, "parallelism": "1 stage x 1 replica",
                   "l2": "no flush: per-step activations exceed the 126 MB L2"},
        "clocks": clocks,
        "e2e": {"value": round(BATCH * steps / (ms_e2e * 1e-3), 2), "unit": "samples/s",
                "h2d_bytes_per_step": host.bytes_per_step, "d2h_bytes_per_step": 4,
                "ms_per_step": round(ms_e2e / steps, 3)},
        "gpu_launches": launches, "entry_point_calls": calls,
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel", "achieved": round(ach, 1),
                     "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": round(ach / pk["bf16_tflops_sustained"], 4), "traffic": None,
                     "kernel_ms_per_step": round(kms / isteps, 3),
                     "note": "contractions only; the step as a whole is bound by the normalisation / "
                             "pointwise kernels' HBM traffic (see model_flops_utilisation)"},
        "model_flops_utilisation": round(FLOPS_PER_SAMPLE * BATCH * steps / (ms * 1e-3) / 1e12 / pk["bf16_tflops_sustained"], 4),
    }
    if with_cpu:
        out["cpu_baseline"] = cpu_baseline()
    return out
