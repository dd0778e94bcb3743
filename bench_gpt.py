"""GPT arm of bench.py (`python bench.py --model gpt`): the 24-layer, hidden-1024, 16-head decoder of the
PipeDream-2BW configuration (sequence 512, vocabulary 50257 padded to 50304), bf16, Adam lr 1.5e-4,
double-buffered weights (at most two versions, one optimizer step per two microbatches), microbatch 8
sequences with uniform token ids.  One GPU: the whole network in one stage; N GPUs under torch.distributed.run:
an N-stage straight pipeline.  Every operator, the attention core included, runs in this repository's kernels."""
import os

import torch

from bench import ClockSampler, one_step, peaks, timed_loop

MICRO = 8
SEQ = 512
METRIC = "gpt24_2bw_train_samples_per_sec"
PARAMS = 405.86e6
# 6 * parameters * tokens (dense layers, forward + backward) + attention score / value products
FLOPS_PER_SAMPLE = 6.0 * (PARAMS - 50304 * 1024 - 512 * 1024) * SEQ + 3 * 24 * 4.0 * SEQ * SEQ * 1024 / 2


class CyclingTokens:
    def __init__(self, batch, device, pool=4, seed=2468):
        from pipedream_b200.stages import SyntheticTokens
        self.items = []
        for x, y in SyntheticTokens(batch, pool, SEQ, 50257, seed=seed):
            self.items.append((x.pin_memory(), y.pin_memory()) if device == "pinned" else (x.to(device), y.to(device)))
        self.bytes_per_step = self.items[0][0].numel() * 8 + self.items[0][1].numel() * 8

    def __iter__(self):
        i = 0
        while True:
            yield self.items[i % len(self.items)]
            i += 1


def build(n_stages, rank, local_rank, backend):
    from pipedream_b200 import adam, runtime, stages
    torch.manual_seed(0)
    pkg = stages.gpt2(n_stages)
    model = pkg.model(torch.nn.CrossEntropyLoss())
    shapes = pkg.boundary_shapes(MICRO)
    dtypes = {k: (torch.int64 if k in ("input0", "target") else torch.bfloat16) for k in shapes}
    if n_stages == 1:
        conf = {"module_to_stage_map": None, "stage_to_rank_map": None, "stage_to_depth_map": None}
    else:
        conf = dict(pkg.conf, stage_to_depth_map=None)
    r = runtime.StageRuntime(
        model=model, distributed_backend=backend, fp16=True, loss_scale=1, training_tensor_shapes=shapes,
        eval_tensor_shapes=dict(shapes), training_tensor_dtypes=dtypes, inputs_module_destinations={"input": 0},
        target_tensor_names={"target"}, configuration_maps=conf,
        master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1") if backend else None, rank=rank, local_rank=local_rank,
        num_ranks_in_server=1, verbose_freq=0, model_type=runtime.IMAGE_CLASSIFICATION)
    opt = adam.AdamWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1,
                                      num_versions=max(2, r.num_warmup_minibatches + 1), lr=1.5e-4, weight_decay=0.01,
                                      macrobatch=True)
    return r, opt


def _line(value, ms, steps, warmup, world, label, clocks, e2e_value, ms_e2e, launches, h2d):
    pk = peaks()
    ach = FLOPS_PER_SAMPLE * value / 1e12 / world
    return {
        "metric": METRIC, "value": round(value, 2), "unit": "samples/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms / steps, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "GPT decoder 24 layers, hidden 1024, 16 heads, sequence 512, vocabulary 50257 (padded to 50304), "
                               "bf16, microbatch 8 sequences of uniform token ids, Adam lr 1.5e-4, 2BW double-buffered weights "
                               "(a step here is one microbatch: forward, backward, optimizer step every second one)",
                   "global_batch": MICRO, "tokens_per_sec": round(value * SEQ, 1), "parallelism": label,
                   "l2": "no flush: weights + activations of a step exceed L2"},
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 2), "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                "ms_per_step": round(ms_e2e / steps, 3)},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel", "achieved": round(ach, 1),
                     "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": round(ach / pk["bf16_tflops_sustained"], 4),
                     "traffic": None, "note": "whole-step model FLOP rate per GPU (6 x parameters x tokens + attention)"},
    }


def run(steps, warmup):
    from pipedream_b200 import _lib
    from pipedream_b200 import functional as pf
    torch.cuda.set_device(0)
    r, opt = build(1, None, 0, None)
    r.train(4 * (steps + warmup) + 16)
    r.set_loader(CyclingTokens(MICRO, "cuda"))
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
    launches = _lib.launches_counted()
    _lib.count_calls(False)
    clocks = sampler.stop()
    host = CyclingTokens(MICRO, "pinned")
    r.set_loader(host)
    ms_e2e = timed_loop(r, opt, steps, 2, True)
    if pf.gemm_poll_error() != 0:
        raise RuntimeError("a tcgen05 kernel reported a bounded wait that ran out")
    return _line(MICRO * steps / (ms * 1e-3), ms, steps, warmup, 1, "1 stage x 1 replica", clocks,
                 MICRO * steps / (ms_e2e * 1e-3), ms_e2e, launches, host.bytes_per_step)


def run_multi(gpus, steps, warmup):
    import torch.distributed as dist
    from bench_multi import run_phase
    from pipedream_b200 import _lib
    from pipedream_b200 import functional as pf
    rank = int(os.environ["RANK"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    world = int(os.environ["WORLD_SIZE"])
    assert world == gpus
    torch.cuda.set_device(local_rank)
    r, opt = build(world, rank, local_rank, "p2p")
    first = r.stage == 0
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    _lib.count_calls(True)
    ms = run_phase(r, opt, CyclingTokens(MICRO, "cuda") if first else None, steps, warmup, False)
    launches = _lib.launches_counted()
    _lib.count_calls(False)
    clocks = sampler.stop() if sampler else None
    host = CyclingTokens(MICRO, "pinned") if first else None
    ms_e2e = run_phase(r, opt, host, steps, 3, True)
    if pf.gemm_poll_error() != 0:
        raise RuntimeError("a tcgen05 kernel reported a bounded wait that ran out")
    t = torch.tensor([ms, ms_e2e, float(launches)], dtype=torch.float64, device="cuda")
    tmax = t.clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    if rank != 0:
        return None
    return _line(MICRO * steps / (tmax[0].item() * 1e-3), tmax[0].item(), steps, warmup, world,
                 "%d-stage straight pipeline" % world, clocks, MICRO * steps / (tmax[1].item() * 1e-3), tmax[1].item(),
                 int(t[2].item()), MICRO * SEQ * 8 + MICRO * SEQ * 8)
