"""GNMT arm of bench.py (`python bench.py --model gnmt`): the 8+8-layer GNMT ("gnmt_large") in bf16,
batch 128 sentence pairs, source/target lengths uniform in [20,50], Zipf(1.1) token ids, label-smoothed
cross-entropy (0.1), Adam lr 2e-3 - all four stages in one process on one GPU."""
import os
import time

import torch

from bench import ClockSampler, peaks

BATCH = 128
METRIC = "gnmt8_train_samples_per_sec"


class CyclingPairs:
    """Endless stream of pre-generated batches; tensors live in pinned host memory (the runtime copies
    them to the device every step, as the reference's loader path does) or already on the device."""

    def __init__(self, batch, device, pool=4, seed=4321):
        from pipedream_b200.stages import SyntheticTranslation
        self.items, self.tokens = [], []
        for (src, sl), (tgt, tl) in SyntheticTranslation(batch, pool, seed=seed):
            if device == "pinned":
                src, tgt = src.pin_memory(), tgt.pin_memory()
            else:
                src, tgt = src.to(device), tgt.to(device)
            self.items.append(((src, sl), (tgt, tl)))
            self.tokens.append(sum(sl) + sum(tl))
        self.bytes_per_step = sum(i[0][0].numel() * 8 + i[1][0].numel() * 8 for i in self.items) // len(self.items)

    def __iter__(self):
        i = 0
        while True:
            yield self.items[i % len(self.items)]
            i += 1


def build(fp16=True, dropout=0.2):
    from pipedream_b200 import adam, gnmt_blocks, runtime, stages
    torch.manual_seed(0)
    model = stages.gnmt_large(dropout=dropout).model(gnmt_blocks.LabelSmoothing(0, 0.1))
    r = runtime.StageRuntime(
        model=model, distributed_backend=None, fp16=fp16, loss_scale=1, training_tensor_shapes={},
        eval_tensor_shapes={}, training_tensor_dtypes={}, inputs_module_destinations={"input0": 0, "input1": 0, "input2": 0},
        target_tensor_names={"target", "target_length"},
        configuration_maps={"module_to_stage_map": None, "stage_to_rank_map": None, "stage_to_depth_map": None},
        master_addr=None, rank=None, local_rank=0, num_ranks_in_server=1, verbose_freq=0,
        model_type=runtime.TRANSLATION)
    opt = adam.AdamWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1, num_versions=1,
                                      lr=2e-3, weight_decay=1e-4)
    return r, opt


def step(r, opt, read_loss=False):
    r.run_forward()
    if read_loss:
        r.loss.item()        # device-to-host read of the step's result
    opt.zero_grad()
    opt.load_old_params()
    r.run_backward()
    opt.load_new_params()
    opt.step()


def loop(r, opt, steps, warmup):
    for _ in range(warmup):
        step(r, opt)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    walls = []
    for _ in range(steps):
        t0 = time.time()
        step(r, opt, True)
        walls.append(round((time.time() - t0) * 1e3, 1))
    e.record()
    torch.cuda.synchronize()
    if os.environ.get("PD_BENCH_DETAIL"):
        print("host ms per step:", walls, file=__import__("sys").stderr)
    return s.elapsed_time(e)


def cpu_baseline(batch=16):
    """The restated reference modules (plain torch) on the host cores: one minibatch of `batch` pairs."""
    from oracle import pipedream_oracle as oracle
    from pipedream_b200 import gnmt_blocks, stages
    torch.manual_seed(0)
    model = stages.gnmt_large().model(gnmt_blocks.LabelSmoothing(0, 0.1))
    mods = [m for (m, _, _) in model[:-1]]
    opt = oracle.StashingOracle("Adam", mods, 1, lr=2e-3, weight_decay=1e-4)
    data = list(stages.SyntheticTranslation(batch, 2))
    t0 = None
    for i, ((src, sl), (tgt, _)) in enumerate(data):
        if i == 1:
            t0 = time.time()
        t = {"input0": src, "input1": torch.LongTensor(sl), "input2": tgt[:-1], "target": tgt[1:].contiguous().view(-1)}
        for (m, ins, outs) in model:
            if outs == ["loss"]:
                t["loss"] = m(t[ins[0]], t["target"])
            else:
                o = m(*[t[n] for n in ins])
                for n, v in zip(outs, o if isinstance(o, tuple) else (o,)):
                    t[n] = v
        opt.zero_grad(); t["loss"].backward(); opt.step()
    dt = time.time() - t0
    return {"value": batch / dt, "unit": "samples/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": "1 minibatch of %d sentence pairs (lengths 20-50), fp32, after 1 untimed minibatch" % batch}


def run(steps, warmup, with_cpu):
    from pipedream_b200 import _lib
    from pipedream_b200 import functional as pf
    torch.cuda.set_device(0)
    r, opt = build()
    r.train(steps + warmup)
    dev_data = CyclingPairs(BATCH, "cuda")
    r.set_loader(dev_data)
    sampler = ClockSampler(0)
    sampler.start()
    # warm up over every batch shape of the pool, so that the caching allocator has stopped growing
    for _ in range(max(warmup, len(dev_data.items) + 1)):
        step(r, opt)
    torch.cuda.synchronize()
    # (1) throughput with device-resident inputs; only the (cheap) call counter is on
    _lib.count_calls(True)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    # The host may run at most two steps ahead of the GPU: with variable-length batches the caching allocator
    # still meets a new size now and then, and a cudaMalloc issued behind a deep launch queue waits for all of
    # it (measured: 100-800 ms stalls when the queue was left unbounded).
    marks = []
    for _ in range(steps):
        if len(marks) >= 2:
            marks.pop(0).synchronize()
        step(r, opt)
        m = torch.cuda.Event()
        m.record()
        marks.append(m)
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e)
    launches, calls = _lib.launches_counted(), dict(_lib.COUNTERS)
    _lib.count_calls(False)
    # (2) a short instrumented pass: CUDA events around every contraction / LSTM time loop.  Several
    # hundred event pairs per step slow the host down, so this pass is not part of any throughput figure.
    isteps = 2
    pf.timeline = pf.ContractionTimeline()
    for _ in range(isteps):
        step(r, opt)
    torch.cuda.synchronize()
    tl = pf.timeline.summary()
    if os.environ.get("PD_BENCH_DETAIL"):
        with open(os.environ["PD_BENCH_DETAIL"], "w") as f:
            for k, v in sorted(pf.timeline.per_shape().items()):
                f.write("%-40s launches/step %5.1f  ms/step %7.3f  TFLOP/s %7.1f\n" % (
                    k, v[0] / isteps, v[2] / isteps, v[1] / max(v[2], 1e-9) / 1e9))
    pf.timeline = None
    clocks = sampler.stop()
    host = CyclingPairs(BATCH, "pinned")
    r.set_loader(host)
    ms_e2e = loop(r, opt, steps, len(host.items) + 1)
    assert pf.gemm_poll_error() == 0
    pk = peaks()
    flops, tms = sum(v[1] for v in tl.values()), sum(v[2] for v in tl.values())
    tok = sum(dev_data.tokens) / len(dev_data.tokens)
    out = {
        "metric": METRIC, "value": round(BATCH * steps / (ms * 1e-3), 2), "unit": "samples/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms / steps, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "GNMT 8+8 layers (hidden 1024, vocab 32320), bf16, batch 128 sentence pairs, lengths "
                               "uniform in [20,50], Zipf(1.1) ids, label smoothing 0.1, Adam lr 2e-3, 4 stages in one process",
                   "global_batch": BATCH, "tokens_per_step": tok, "tokens_per_sec": round(tok * steps / (ms * 1e-3), 1),
                   "parallelism": "1 GPU", "l2": "no flush: weights + activations of a step exceed L2"},
        "clocks": clocks,
        "e2e": {"value": round(BATCH * steps / (ms_e2e * 1e-3), 2), "unit": "samples/s",
                "h2d_bytes_per_step": host.bytes_per_step, "d2h_bytes_per_step": 8, "ms_per_step": round(ms_e2e / steps, 3)},
        "gpu_launches": launches, "entry_point_calls": calls,
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel", "achieved": round(flops / max(tms, 1e-9) / 1e9, 1),
                     "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": round(flops / max(tms, 1e-9) / 1e9 / pk["bf16_tflops_sustained"], 4), "traffic": None,
                     "kernel_ms_per_step": round(tms / isteps, 3),
                     "note": "lstm_fwd / lstm_bwd entries time the whole time loop (recurrent contraction + cell kernel per step)",
                     "by_pass": {k: {"tflops": round(v[1] / max(v[2], 1e-9) / 1e9, 1), "ms_per_step": round(v[2] / isteps, 3)}
                                 for k, v in sorted(tl.items())}},
    }
    if with_cpu:
        out["cpu_baseline"] = cpu_baseline()
    return out


def partition_for(n):
    """(module_to_stage_map, stage_to_rank_map, label) of the multi-GPU GNMT runs: N=2 two stages (encoder half /
    decoder half), N=4 the reference's four-stage split, N=8 the same four stages with two replicas each."""
    if n == 2:
        return [0, 0, 1, 1, 1], {0: [0], 1: [1]}, "2-stage pipeline"
    if n == 4:
        return [0, 1, 2, 3, 3], {s: [s] for s in range(4)}, "4-stage pipeline"
    if n == 8:
        return [0, 1, 2, 3, 3], {s: [2 * s, 2 * s + 1] for s in range(4)}, "4-stage pipeline x 2 replicas"
    raise ValueError("GNMT multi-GPU partitions exist for 2, 4 and 8 GPUs")


def run_multi(gpus, steps, warmup):
    """One process per GPU (torch.distributed.run): stages over NVLink peer channels, replicas over NCCL."""
    import torch.distributed as dist
    from bench_multi import run_phase
    from pipedream_b200 import _lib, adam, gnmt_blocks, runtime, stages
    from pipedream_b200 import functional as pf
    rank = int(os.environ["RANK"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    world = int(os.environ["WORLD_SIZE"])
    assert world == gpus, "launch with torch.distributed.run --nproc-per-node %d" % gpus
    torch.cuda.set_device(local_rank)
    m2s, s2r, label = partition_for(world)
    torch.manual_seed(0)
    model = stages.gnmt_large(dropout=0.2).model(gnmt_blocks.LabelSmoothing(0, 0.1))
    B, Tm, H, V = BATCH, 50, 1024, 32320
    shapes = {"input0": (Tm, B), "input1": (B,), "input2": (Tm, B), "target": (Tm * B,), "target_length": (B,),
              "out0": (Tm, B, H), "out1": (Tm, B, H), "out12": (Tm, B, H), "out13": (Tm, B, H), "out14": (Tm, B, H),
              "out15": (Tm, B, 2 * H), "out12again": (Tm, B, H), "out18": (Tm, B, V)}
    dtypes = {k: torch.bfloat16 for k in shapes}
    dtypes.update({k: torch.int64 for k in ("input0", "input1", "input2", "target", "target_length")})
    conf = {"module_to_stage_map": m2s, "stage_to_rank_map": s2r, "stage_to_depth_map": None}
    r = runtime.StageRuntime(
        model=model, distributed_backend="p2p", fp16=True, loss_scale=1, training_tensor_shapes=shapes,
        eval_tensor_shapes=dict(shapes), training_tensor_dtypes=dtypes,
        inputs_module_destinations={"input0": 0, "input1": 1, "input2": 1},
        target_tensor_names={"target", "target_length"}, configuration_maps=conf,
        master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1"), rank=rank, local_rank=local_rank,
        num_ranks_in_server=1, verbose_freq=0, model_type=runtime.TRANSLATION)
    opt = adam.AdamWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1,
                                      num_versions=r.num_warmup_minibatches + 1, lr=2e-3, weight_decay=1e-4)
    first = r.stage == 0
    # this stage's share of the work per minibatch, for the stage roofline: every weight matrix (embedding tables
    # aside, which are gathered, not multiplied) is used once per token forward and twice backward; Adam with an
    # fp32 master copy moves 30 bytes per parameter, the three passes read the bf16 weights once each; an LSTM
    # layer keeps gate activations and cell states per token for its backward pass (about 30 H bytes in all)
    mat = sum(p.numel() for m in r.modules() for n_, p in m.named_parameters() if p.dim() >= 2 and "embed" not in n_)
    allp = sum(p.numel() for p in r.parameters())
    tokens = BATCH * 35.0
    work = {"stage": r.stage, "rank": rank, "tflop": 6.0 * mat * tokens / 1e12,
            "hbm_gb": (allp * 36.0 + mat / (8.0 * H) * tokens * 30.0 * 2) / 1e9}
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    # the untimed head of the phase (>= 6 minibatches) covers every batch shape of the pool (allocator growth)
    dev = CyclingPairs(BATCH, "cuda", seed=4321 + 1000 * rank) if first else None
    _lib.count_calls(True)
    # with R replicas per stage every rank's minibatch count must be a multiple of R (round-robin routing)
    reps = len(s2r[0])
    even = lambda w: w + (-(steps + w)) % reps
    ms = run_phase(r, opt, dev, steps, even(max(warmup, 6)), False)
    launches = _lib.launches_counted()
    _lib.count_calls(False)
    clocks = sampler.stop() if sampler else None
    host = CyclingPairs(BATCH, "pinned", seed=4321 + 1000 * rank) if first else None
    ms_e2e = run_phase(r, opt, host, steps, even(3), True)
    if pf.gemm_poll_error() != 0:
        raise RuntimeError("a tcgen05 kernel reported a bounded wait that ran out")
    t = torch.tensor([ms, ms_e2e, float(launches)], dtype=torch.float64, device="cuda")
    tmax = t.clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    r0 = len(s2r[0])
    work["ms_own"] = ms / steps * len(s2r[r.stage]) / r0          # measured period per minibatch of this replica
    sent = [n for n in r.send_ranks if n in dtypes and dtypes[n].is_floating_point]
    work["nvlink_mb"] = 2 * sum(35.0 * BATCH * shapes[n][-1] * 2 for n in sent) / 1e6     # activations + gradients
    works = [None] * world
    dist.all_gather_object(works, work)
    if rank != 0:
        return None
    pk = peaks()
    stage_roofline = []
    for w in sorted(works, key=lambda w: (w["stage"], w["rank"])):
        if w["rank"] != s2r[w["stage"]][0]:
            continue
        t_s = max(w["tflop"] / pk["bf16_tflops_sustained"], w["hbm_gb"] / pk["hbm_gbs"]) + w["nvlink_mb"] / 1e3 / 770.0
        stage_roofline.append({"stage": w["stage"], "replicas": len(s2r[w["stage"]]), "tflop_per_minibatch": round(w["tflop"], 3),
                               "hbm_gb_per_minibatch": round(w["hbm_gb"], 3), "nvlink_mb_per_minibatch": round(w["nvlink_mb"], 1),
                               "roofline_ms": round(t_s * 1e3, 3), "measured_ms": round(w["ms_own"], 3),
                               "frac": round(t_s * 1e3 / w["ms_own"], 4)})
    samples = BATCH * r0 * steps
    return {
        "metric": METRIC, "value": round(samples / (tmax[0].item() * 1e-3), 2), "unit": "samples/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": round(tmax[0].item() / steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "GNMT 8+8 layers (hidden 1024, vocab 32320), bf16, batch 128 sentence pairs per stage-0 "
                               "replica, lengths uniform in [20,50], Zipf(1.1) ids, label smoothing 0.1, Adam lr 2e-3, "
                               "1F1B with weight stashing", "global_batch": BATCH * r0, "parallelism": label,
                   "l2": "no flush: weights + activations of a step exceed L2"},
        "clocks": clocks,
        "e2e": {"value": round(samples / (tmax[1].item() * 1e-3), 2), "unit": "samples/s",
                "h2d_bytes_per_step": (dev.bytes_per_step if dev else 0) * r0, "d2h_bytes_per_step": 8 * len(s2r[max(s2r)]),
                "ms_per_step": round(tmax[1].item() / steps, 3)},
        "gpu_launches": int(t[2].item()),
        "stage_roofline": stage_roofline,
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel", "achieved": None, "peak": peaks()["bf16_tflops_sustained"],
                     "unit": "TFLOP/s", "frac": None, "traffic": None,
                     "note": "per-kernel figures are reported by the 1-GPU run (python bench.py --model gnmt)"},
    }
