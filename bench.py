"""Throughput benchmark of the pipeline-parallel training step (VGG-16, bf16, synthetic data).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N = 1: the whole of VGG-16 in one stage on one GPU, batch 64 (the per-replica batch of the
hybrid configuration the metric is quoted on).  N > 1 (under torch.distributed.run): the same
network as a 2-stage pipeline cut after the flatten, stage 0 (all convolutions) replicated on
N-1 GPUs and stage 1 (the three Linear layers) on one; every replica of stage 0 takes batch 64.

One JSON line is printed by rank 0.  `value` is samples/s with the inputs already resident in
HBM; `e2e` is the same loop fed from pinned host memory with the loss read back every step.
`--impl reference` times the CPU oracle (the restatement of the reference's own Python/PyTorch
path; the reference itself cannot travel to the benchmark machine) on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

BATCH = 64
METRIC = "vgg16_train_samples_per_sec"
UNIT = "samples/s"
# algorithmic FLOPs of one VGG-16 training sample (2 per multiply-add; forward 30.94 G,
# backward 61.71 G, counted on the reference modules with torch.utils.flop_counter)
FLOPS_PER_SAMPLE = 92.65e9


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def measured_traffic():
    """DRAM traffic per launch of the contraction kernel as ncu measured it, read from the committed profile
    summary.  The summary names the sha256 of the kernel source it was taken on; if the source has changed since,
    the figure is stale and None is reported instead."""
    import hashlib
    import re
    path = os.path.join(ROOT, "profiles", "gemm_tcgen05_conv_56x56_256_ncu.md")
    src = os.path.join(ROOT, "pipedream_b200", "csrc", "pd_gemm_sm100.cu")
    try:
        text = open(path).read()
        sha = hashlib.sha256(open(src, "rb").read()).hexdigest()
    except OSError:
        return None, "no profile summary"
    m = re.search(r"kernel_source_sha256:\s*([0-9a-f]{64})", text)
    t = re.search(r"dram_bytes_per_launch_mean:\s*([0-9.eE+]+)", text)
    c = re.search(r"captured_at_commit:\s*([0-9a-f]+)", text)
    if not (m and t):
        return None, "profile summary carries no machine-readable traffic line"
    if m.group(1) != sha:
        return None, "kernel source changed since the capture (commit %s)" % (c.group(1) if c else "?")
    return float(t.group(1)), "ncu capture at commit %s: conv 64x56x56 256->256, mean of fwd/dgrad/wgrad; algorithmic 221.6e6" % (
        c.group(1) if c else "?")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm.sort()
        # median of the samples under load (upper half: idle samples at the edges are dropped)
        load = sm[len(sm) // 2:]
        return {"sm_mhz": load[len(load) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


class CyclingLoader:
    """Endless (images, labels) stream from a small pool of pre-generated batches.
    device="cuda": batches already resident in HBM; device="pinned": pinned host memory, so
    the consumer's .to(device) is a real host-to-device copy every step."""

    def __init__(self, batch, device, pool=4, seed=1234):
        from pipedream_b200.stages import SyntheticImages
        self.items = []
        for x, y in SyntheticImages(batch, pool, seed=seed):
            if device == "pinned":
                self.items.append((x.pin_memory(), y.pin_memory()))
            else:
                self.items.append((x.to(device), y.to(device)))
        self.bytes_per_step = self.items[0][0].numel() * 4 + self.items[0][1].numel() * 8

    def __iter__(self):
        i = 0
        while True:
            yield self.items[i % len(self.items)]
            i += 1


def build_single_stage(fp16=True):
    """StageRuntime + optimizer for all of VGG-16 on cuda:0, built the way the driver script does
    (runtime/image_classification/main_with_runtime.py:129-229)."""
    from pipedream_b200 import runtime, sgd, stages
    torch.manual_seed(0)
    pkg = stages.vgg16("gpus=1")
    model = pkg.model(torch.nn.CrossEntropyLoss())
    shapes = {"input0": (BATCH, 3, 224, 224), "target": (BATCH,), "out0": (BATCH, 1000)}
    dtypes = {"input0": torch.int64, "target": torch.int64, "out0": torch.bfloat16 if fp16 else torch.float32}
    r = runtime.StageRuntime(
        model=model, distributed_backend=None, fp16=fp16, loss_scale=1, training_tensor_shapes=shapes,
        eval_tensor_shapes=dict(shapes), training_tensor_dtypes=dtypes, inputs_module_destinations={"input": 0},
        target_tensor_names={"target"},
        configuration_maps={"module_to_stage_map": None, "stage_to_rank_map": None, "stage_to_depth_map": None},
        master_addr=None, rank=None, local_rank=0, num_ranks_in_server=1, verbose_freq=0,
        model_type=runtime.IMAGE_CLASSIFICATION)
    opt = sgd.SGDWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1,
                                    num_versions=r.num_warmup_minibatches + 1, lr=0.01, momentum=0.9,
                                    weight_decay=5e-4)
    return r, opt


def one_step(r, opt, read_loss):
    """One minibatch of the 1F1B loop of a stage without warm-up (main_with_runtime.py:363-413)."""
    r.run_forward()
    loss = r.loss.item() if read_loss else None
    opt.zero_grad()
    opt.load_old_params()
    r.run_backward()
    opt.load_new_params()
    opt.step()
    return loss


def timed_loop(r, opt, steps, warmup, read_loss):
    """W untimed steps, then K steps between CUDA events; returns milliseconds for the K steps."""
    for _ in range(warmup):
        one_step(r, opt, read_loss)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        one_step(r, opt, read_loss)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end)


def cpu_baseline(sample_steps=3, batch=8):
    """The CPU oracle (port of the reference's PyTorch path) on the host cores, fp32, on a bounded
    sample of the workload: `sample_steps` minibatches of `batch` images after one untimed one."""
    from oracle import pipedream_oracle as oracle
    from pipedream_b200.stages import SyntheticImages
    torch.set_num_threads(os.cpu_count() or 1)
    torch.manual_seed(0)
    st = oracle.vgg16_stages(None)
    model = [(st[0], ["input0"], ["out0"]), (torch.nn.CrossEntropyLoss(), ["out0"], ["loss"])]
    pipe = oracle.PipelineOracle(model, [0, 0], {0: [0]}, None, "SGD", dict(lr=0.01, momentum=0.9, weight_decay=5e-4))
    pipe.run({0: SyntheticImages(batch, 1)}, 1)
    t0 = time.time()
    pipe.run({0: SyntheticImages(batch, sample_steps, seed=99)}, sample_steps)
    dt = time.time() - t0
    return {"value": batch * sample_steps / dt, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": "%d minibatches of %d images, fp32, whole VGG-16 in one stage, after 1 untimed minibatch"
                      % (sample_steps, batch)}


def run_gpu_single(steps, warmup):
    """N = 1: whole VGG-16, batch 64, bf16, one stage on cuda:0."""
    from pipedream_b200 import _lib
    from pipedream_b200 import functional as pf
    torch.cuda.set_device(0)
    r, opt = build_single_stage(fp16=True)
    r.train(steps + warmup)

    # (1) device-resident inputs: `value`
    r.set_loader(CyclingLoader(BATCH, "cuda"))
    sampler = ClockSampler(0)
    sampler.start()
    _lib.count_calls(True)
    for _ in range(warmup):
        one_step(r, opt, False)
    torch.cuda.synchronize()
    _lib.count_calls(True)                      # restart the count for the timed region
    pf.timeline = pf.ContractionTimeline()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        one_step(r, opt, False)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    launches = _lib.launches_counted()
    calls = dict(_lib.COUNTERS)
    _lib.count_calls(False)
    tl = pf.timeline.summary()
    if os.environ.get("PD_BENCH_DETAIL"):
        with open(os.environ["PD_BENCH_DETAIL"], "w") as f:
            for k, v in sorted(pf.timeline.per_shape().items()):
                f.write("%-40s launches/step %3d  ms/step %7.3f  TFLOP/s %7.1f\n" % (
                    k, v[0] // steps, v[2] / steps, v[1] / max(v[2], 1e-9) / 1e9))
    pf.timeline = None
    clocks = sampler.stop()

    # (2) pinned host inputs + loss read back every step: `e2e`
    host = CyclingLoader(BATCH, "pinned")
    r.set_loader(host)
    ms_e2e = timed_loop(r, opt, steps, max(1, warmup // 2), True)
    err = pf.gemm_poll_error()
    if err != 0:
        raise RuntimeError("a tcgen05 kernel reported a bounded wait that ran out (code %d)" % err)

    pk = peaks()
    traffic, traffic_note = measured_traffic()
    tot_flops = sum(v[1] for v in tl.values())
    tot_ms = sum(v[2] for v in tl.values())
    n_launch = sum(v[0] for v in tl.values())
    achieved = tot_flops / (tot_ms * 1e-3) / 1e12 if tot_ms > 0 else 0.0
    roof = {
        "bound": "tensor", "kernel": "gemm_tcgen05_kernel", "achieved": round(achieved, 1),
        "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": round(achieved / pk["bf16_tflops_sustained"], 4),
        "peak_source": pk["source"] + " (sustained cuBLAS bf16)",
        "traffic": traffic, "traffic_case": traffic_note,
        "launches_per_step": n_launch // max(1, steps), "kernel_ms_per_step": round(tot_ms / steps, 3),
        "algorithmic_tflop_per_step": round(tot_flops / steps / 1e12, 3),
        "by_pass": {k: {"launches": v[0] // max(1, steps), "tflops": round(v[1] / (v[2] * 1e-3) / 1e12, 1),
                        "ms_per_step": round(v[2] / steps, 3)} for k, v in sorted(tl.items()) if v[2] > 0},
    }
    return {
        "metric": METRIC, "value": round(BATCH * steps / (ms * 1e-3), 2), "unit": UNIT, "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "VGG-16 (13 conv3x3 + 3 FC, 1000 classes) bf16 training step, batch 64 of 3x224x224 "
                               "N(0,1) images, SGD momentum 0.9 lr 0.01 wd 5e-4, one stage on one GPU",
                   "global_batch": BATCH, "parallelism": "1 stage x 1 replica",
                   "l2": "no flush: per-step activations (>1 GB) exceed the 126 MB L2"},
        "clocks": clocks,
        "e2e": {"value": round(BATCH * steps / (ms_e2e * 1e-3), 2), "unit": UNIT,
                "h2d_bytes_per_step": host.bytes_per_step, "d2h_bytes_per_step": 4,
                "ms_per_step": round(ms_e2e / steps, 3)},
        "gpu_launches": launches, "entry_point_calls": calls,
        "roofline": roof,
        "model_flops_utilisation": round(FLOPS_PER_SAMPLE * BATCH * steps / (ms * 1e-3) / 1e12 / pk["bf16_tflops_sustained"], 4),
    }


def reference_partition(n_gpus):
    """The stage / replica layout the GPU arm uses at this GPU count, for the CPU arm to follow."""
    if n_gpus <= 1:
        return None, [0, 0], {0: [0]}, "1 stage x 1 replica"
    if n_gpus == 2:
        return None, [0, 0], {0: [0, 1]}, "1 stage x 2 replicas (data parallel)"
    return "flatten", [0, 1, 1], {0: list(range(n_gpus - 1)), 1: [n_gpus - 1]}, "hybrid %d:1" % (n_gpus - 1)


def run_reference(steps, warmup, n_gpus):
    """--impl reference: the reference's CPU path on the host cores - the oracle port, because the reference is
    Python source that cannot travel to the benchmark machine - for the same metric, network and stage / replica
    layout as the GPU arm at this GPU count.  All ranks of the layout are stepped inside one process (the oracle's
    pipeline simulation: 1F1B with weight stashing, replica gradient averaging) with every host thread given to
    torch's intra-op pool; each step is a bounded sample: one minibatch of 8 images (instead of 64) per stage-0
    replica, fp32.  Under torch.distributed.run rank 0 alone runs it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    from oracle import pipedream_oracle as oracle
    from pipedream_b200.stages import SyntheticImages
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)          # the launcher exports OMP_NUM_THREADS=1 for its workers
    batch = 8
    cut, m2s, s2r, label = reference_partition(n_gpus)
    torch.manual_seed(0)
    st = oracle.vgg16_stages(cut)
    if len(st) == 1:
        model = [(st[0], ["input0"], ["out0"]), (torch.nn.CrossEntropyLoss(), ["out0"], ["loss"])]
    else:
        model = [(st[0], ["input0"], ["out0"]), (st[1], ["out0"], ["out1"]), (torch.nn.CrossEntropyLoss(), ["out1"], ["loss"])]
    r0 = len(s2r[0])
    # a multi-rank CPU step costs r0 minibatches: keep the whole run within a few minutes
    steps_run = max(2, min(steps, max(2, 24 // r0)))
    warm_run = min(warmup, 1 if r0 > 1 else 2)
    pipe = oracle.PipelineOracle(model, m2s, s2r, None, "SGD", dict(lr=0.01, momentum=0.9, weight_decay=5e-4, scale_lr=True))
    if warm_run > 0:
        pipe.run({k: SyntheticImages(batch, warm_run, seed=7 + k) for k in s2r[0]}, warm_run)
    t0 = time.time()
    pipe.run({k: SyntheticImages(batch, steps_run, seed=99 + k) for k in s2r[0]}, steps_run)
    dt = time.time() - t0
    v = round(batch * r0 * steps_run / dt, 3)
    sample = ("%d timed steps (of the %d asked for) after %d untimed; each step = one minibatch of %d images (instead of 64) "
              "per stage-0 replica, fp32, layout %s simulated rank by rank in one process, %d intra-op threads"
              % (steps_run, steps, warm_run, batch, label, cores))
    return {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": n_gpus, "steps": steps_run,
        "warmup": warm_run, "ms_per_step": round(dt / steps_run * 1e3, 1), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "VGG-16 training step on host cores (CPU restatement of the reference's PyTorch path)",
                   "global_batch": batch * r0, "parallelism": label},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def secondary_gnmt_single(steps, warmup):
    """The other network of the headline metric on the same GPU right after VGG-16: GNMT 8+8 layers, batch 128,
    the four stages in one process.  A trimmed copy of `python bench.py --model gnmt`."""
    import gc
    import bench_gnmt
    gc.collect()
    torch.cuda.empty_cache()
    try:
        g = bench_gnmt.run(steps, warmup, False)
    except Exception as e:      # the headline line must not be lost to the secondary run
        return {"error": "%s: %s" % (type(e).__name__, e)}
    keep = ("metric", "value", "unit", "steps", "warmup", "ms_per_step", "dtype", "e2e", "gpu_launches")
    out = {k: g[k] for k in keep if k in g}
    out["config"] = {k: g["config"][k] for k in ("workload", "global_batch", "tokens_per_sec", "parallelism")}
    out["roofline"] = {k: g["roofline"][k] for k in ("bound", "kernel", "achieved", "peak", "unit", "frac", "kernel_ms_per_step")}
    return out


def run_profile_case_other(name):
    """A few launches of one of the memory-bound kernels on a case that exceeds L2 but stays under 1 GB, for `ncu`
    captures; prints the kernel's algorithmic bytes per launch (what its roofline fraction is measured against):
    sgd / adam : the fused optimizer over a 2-version ring, 64 M bf16 parameters with fp32 master copy;
    softmax_ce : criterion forward + backward on [6400, 32320] bf16 logits (GNMT: 50 steps x 128 pairs);
    sdpa       : causal self-attention core forward + backward, 16 x 16 heads x 512 tokens x 64;
    pool       : 2x2 max-pool forward, backward fused with the bias-gradient sums, the sums alone, the first layer's
                 patch matrix, on a [16, 64, 224, 224] bf16 activation;
    bn         : BatchNorm2d training forward + backward on a padded-NHWC [64, 58, 58, 256] bf16 tensor;
    layernorm  : LayerNorm forward + backward on [65536, 1024] bf16 rows;
    lstm       : one LSTM layer's recurrence, T = 50, B = 128, H = 1024, forward + backward;
    attn       : normalised additive attention forward + backward, B = 128, Tq = Tk = 50, 1024 channels."""
    import ctypes
    from pipedream_b200 import functional as pf
    from pipedream_b200._lib import call
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(0)
    bf = torch.bfloat16
    info = {"case": name}
    if name in ("sgd", "adam"):
        n, V = 64 * 1024 * 1024, 2
        arena = torch.zeros(V, n, device="cuda", dtype=bf)
        master = torch.randn(n, device="cuda") * 0.01
        grad = torch.randn(n, device="cuda") * 0.01
        sa, sb = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        for i in range(4):
            if name == "sgd":
                call("pd_opt_sgd_multi_tensor", p(arena), n, i % 2, (i + 1) % 2, 1, p(master), p(grad), p(sa), n, 0.01, 0.9, 0.0,
                     5e-4, 0, int(i == 0), 1.0, st)
            else:
                call("pd_opt_adam_multi_tensor", p(arena), n, i % 2, (i + 1) % 2, 1, p(master), p(grad), p(sa), p(sb), n, 2e-3,
                     0.9, 0.999, 1e-8, 1e-4, i + 1, 1.0, st)
        # read gradient, master (and the moments); write master, moments and the bf16 weights of the new version
        info["algorithmic_bytes_per_launch"] = n * (4 + 4 + 4 + 4 + 4 + 2) if name == "sgd" else n * (4 + 4 + 4 + 4 + 4 + 4 + 4 + 2)
    elif name == "softmax_ce":
        rows, C = 6400, 32320
        logits = (torch.randn(rows, C, generator=g) * 2).cuda().to(bf)
        target = torch.randint(1, C, (rows,), generator=g).cuda()
        up = torch.ones((), device="cuda")
        for _ in range(3):
            loss, lse, _ = pf.softmax_ce_fwd(logits, target, 0.1, 0, 1.0)
            pf.softmax_ce_bwd(logits, target, lse, 0.1, 0, up, 1.0)
        info["algorithmic_bytes_per_launch"] = {"forward (read logits)": rows * C * 2, "backward (read logits, write gradient)": rows * C * 4}
    elif name == "pool":
        # conv1_2's output of VGG-16 at a quarter of the batch: [16, 226, 226, 64] bf16 (105 MB) and its pooled gradient
        N, H, C = 16, 224, 64
        x = pf.pack_pnhwc(torch.randn(N, C, H, H, generator=g).cuda().to(bf).relu())
        dy = pf.pack_pnhwc(torch.randn(N, C, H // 2, H // 2, generator=g).cuda().to(bf))
        img = torch.randn(N, 3, H, H, generator=g).cuda()
        cs = torch.zeros(C, device="cuda")
        for _ in range(3):
            pf.maxpool2_fwd(x, False)
            dx, part = pf.maxpool2_bwd_colsum(x, dy, True)
            pf.colsum_finish(part, cs, False)
            pf.relu_bwd_colsum(dx, None, None, cs, False)
            pf.im2col3x3(img, 32, bf)
        info["algorithmic_bytes_per_launch"] = {
            "maxpool2_fwd (read x, write y)": x.numel() * 2 + dy.numel() * 2,
            "maxpool2_bwd_colsum (read x and dy, write dx)": 2 * x.numel() * 2 + dy.numel() * 2,
            "relu_bwd_colsum, sums only (read dy)": x.numel() * 2,
            "im2col3x3 (read the images, write 64-byte patch rows)": img.numel() * 4 + N * (H + 2) * (H + 2) * 64}
    elif name == "sdpa":
        # the attention core of a GPT block: 16 sequences x 16 heads x 512 tokens x 64 (attention weights: 134 MB)
        B, H, T, d = 16, 16, 512, 64
        qkv = (torch.randn(B, T, 3 * H * d, generator=g) * 0.8).cuda().to(bf)
        dout = torch.randn(B, T, H * d, generator=g).cuda().to(bf)
        for _ in range(3):
            out, probs = pf.sdpa_causal_fwd(qkv, H)
            pf.sdpa_causal_bwd(qkv, probs, dout, H)
        info["algorithmic_bytes_per_launch"] = {
            "S = Q K^T / dP = dO V^T (write the lower tiles of the T x T matrix)": B * H * T * T * 2 * 5 // 8,
            "causal softmax rows (read and write the lower triangle, write zeros above)": B * H * T * T * 2 * 3 // 2,
            "P V / dS K / P^T dO / dS^T Q (read the lower tiles)": B * H * T * T * 2 * 5 // 8}
        info["algorithmic_flops"] = {"forward": 4 * B * H * T * T * d // 2, "backward": 10 * B * H * T * T * d // 2}
    elif name == "bn":
        N, H, C = 64, 56, 256
        x = pf.pack_pnhwc(torch.randn(N, C, H, H, generator=g).cuda().to(bf))
        dy = pf.pack_pnhwc(torch.randn(N, C, H, H, generator=g).cuda().to(bf))
        gamma, beta = torch.ones(C, device="cuda", dtype=bf), torch.zeros(C, device="cuda", dtype=bf)
        rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
        dg, db = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
        for _ in range(3):
            y, mean, invstd = pf.bn_fwd(x, gamma, beta, 1e-5, 0.1, True, rm, rv)
            pf.bn_bwd(x, dy, y, gamma, mean, invstd, dg, db, False)
        info["algorithmic_bytes_per_launch"] = {"tensor": x.numel() * 2, "forward": "read x twice, write y", "backward": "read x, dy, y twice, write dx"}
    elif name == "layernorm":
        rows, C = 65536, 1024
        x = torch.randn(rows, C, generator=g).cuda().to(bf)
        dy = torch.randn(rows, C, generator=g).cuda().to(bf)
        gamma, beta = torch.ones(C, device="cuda", dtype=bf), torch.zeros(C, device="cuda", dtype=bf)
        dg, db = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
        for _ in range(3):
            y, mean, rstd = pf.layernorm_fwd(x, gamma, beta, 1e-5)
            pf.layernorm_bwd(x, dy, gamma, mean, rstd, dg, db, False)
        info["algorithmic_bytes_per_launch"] = {"forward": rows * C * 4, "backward": rows * C * 6}
    elif name == "lstm":
        T, B, H = 50, 128, 1024
        gx = (torch.randn(T, B, 4 * H, generator=g) * 0.1).cuda().to(bf)
        w = (torch.randn(4 * H, H, generator=g) * 0.03).cuda().to(bf)
        b = torch.zeros(4 * H, device="cuda", dtype=bf)
        dyy = (torch.randn(T, B, H, generator=g) * 0.1).cuda().to(bf)
        for _ in range(2):
            y, act, c_all = pf.lstm_fwd(gx, w, b, T, B, H)
            pf.lstm_bwd(dyy, w, act, c_all)
        info["algorithmic_flop_per_launch"] = 2.0 * (T - 1) * B * 4 * H * H
        info["steps"] = T
    elif name == "attn":
        B, T, n = 128, 50, 1024
        pq = (torch.randn(B, T, n, generator=g) * 0.3).cuda().to(bf)
        pk = (torch.randn(B, T, n, generator=g) * 0.3).cuda().to(bf)
        keys = (torch.randn(T, B, n, generator=g) * 0.3).cuda().to(bf)
        v = (torch.randn(n, generator=g) * 0.05).cuda()
        nb = torch.zeros(n, device="cuda", dtype=bf)
        lens = torch.full((B,), T, dtype=torch.int64, device="cuda")
        dctx = (torch.randn(T, B, n, generator=g) * 0.1).cuda().to(bf)
        for _ in range(2):
            probs, ctx = pf.attn_fwd(pq, pk, keys, v, nb, lens)
            pf.attn_bwd(pq, pk, keys, v, nb, probs, dctx)
        info["tanh_per_pass"] = B * T * T * n
    else:
        raise ValueError(name)
    torch.cuda.synchronize()
    print(json.dumps(info))


def run_profile_case(name):
    """A few launches of one contraction at one layer shape, for `ncu` captures of the tensor-core kernel on
    a case that is larger than L2 but well under 1 GB:
    fwd|dgrad|wgrad : batch 64, 56x56, 256 -> 256 channels, bf16 (a tensor-bound layer);
    narrow_fwd|narrow_dgrad : batch 16, 224x224, 64 -> 64 channels (a layer bound by shared-memory fill);
    patch_fwd : the first layer's patch-matrix contraction, [16*226*226, 32] x [64, 32]^T with bias + ReLU."""
    from pipedream_b200 import functional as pf
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(0)
    if name.startswith("narrow"):
        N, H, W, Cin, Cout = 16, 224, 224, 64, 64
    elif name == "patch_fwd":
        N, H, W, Cin, Cout = 16, 224, 224, 3, 64
    else:
        N, H, W, Cin, Cout = 64, 56, 56, 256, 256
    bias = torch.zeros(Cout, device="cuda", dtype=torch.bfloat16)
    if name == "patch_fwd":
        col = torch.randn(N * (H + 2) * (W + 2), 32, generator=g).cuda().to(torch.bfloat16)
        w = (torch.randn(Cout, 32, generator=g) * 0.1).cuda().to(torch.bfloat16)
        for _ in range(4):
            pf.gemm_nt(col, w, bias=bias, relu=True, pad_hw=(H + 2, W + 2))
        torch.cuda.synchronize()
        assert pf.gemm_poll_error() == 0
        print(json.dumps({"case": name, "shape": [col.shape[0], Cout, 32],
                          "algorithmic_flop_per_launch": 2.0 * N * H * W * 27 * Cout,
                          "algorithmic_bytes_per_launch": int(col.numel() * 2 + col.shape[0] * Cout * 2)}))
        return
    x = pf.pack_pnhwc(torch.randn(N, Cin, H, W, generator=g).cuda().to(torch.bfloat16))
    dy = pf.pack_pnhwc(torch.randn(N, Cout, H, W, generator=g).cuda().to(torch.bfloat16))
    w = (torch.randn(Cout, 9 * Cin, generator=g) * 0.02).cuda().to(torch.bfloat16)
    dw = torch.zeros(Cout, 9 * Cin, device="cuda")
    for _ in range(4):
        if name.endswith("fwd"):
            pf.conv2d_fwd(x, w, 9 * Cin, Cout, bias, True)
        elif name.endswith("dgrad"):
            pf.conv2d_dgrad(dy, w, 9 * Cin, Cin, relu_aux=x)
        else:
            pf.conv2d_wgrad(x, dy, dw, 9 * Cin, accumulate=False)
    torch.cuda.synchronize()
    assert pf.gemm_poll_error() == 0
    flops = 18.0 * N * H * W * Cin * Cout
    print(json.dumps({"case": name, "shape": [N, H, W, Cin, Cout], "algorithmic_flop_per_launch": flops,
                      "algorithmic_bytes_per_launch": int(x.numel() * 2 + dy.numel() * 2 + w.numel() * 2)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed steps (default: 200 for the GPU arm, 20 for --impl reference)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the GNMT run that the default line carries under \"secondary\"")
    ap.add_argument("--model", default="vgg16", choices=["vgg16", "gnmt", "resnet50", "gpt"],
                    help="vgg16 (default, the headline line), gnmt (8+8-layer GNMT), resnet50 or gpt (24-layer 2BW decoder)")
    ap.add_argument("--profile-case", default=None,
                    choices=["fwd", "dgrad", "wgrad", "narrow_fwd", "narrow_dgrad", "patch_fwd", "sgd", "adam", "softmax_ce", "pool", "sdpa", "bn",
                             "layernorm", "lstm", "attn"],
                    help="run a few launches of one kernel family on a small case (for ncu) and exit")
    a = ap.parse_args()
    if a.profile_case in ("sgd", "adam", "softmax_ce", "pool", "sdpa", "bn", "layernorm", "lstm", "attn"):
        run_profile_case_other(a.profile_case)
        return
    if a.profile_case:
        run_profile_case(a.profile_case)
        return
    if a.steps is None:
        a.steps = 20 if a.impl == "reference" else 200
    if a.impl == "reference":
        out = run_reference(a.steps, a.warmup, a.gpus)
        if out is not None:
            print(json.dumps(out))
        return
    if a.warmup < 3:
        a.warmup = 3
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if a.model == "gnmt" and a.gpus == 1 and world == 1:
        import bench_gnmt
        print(json.dumps(bench_gnmt.run(a.steps, a.warmup, not a.no_cpu_baseline)))
        return
    if a.model == "gnmt":
        import bench_gnmt
        import torch.distributed as dist
        out = bench_gnmt.run_multi(a.gpus, a.steps, a.warmup)
        if out is not None:
            print(json.dumps(out), flush=True)
        if dist.is_initialized():
            dist.destroy_process_group()
        return
    if a.model == "gpt":
        import bench_gpt
        if a.gpus == 1 and world == 1:
            print(json.dumps(bench_gpt.run(a.steps, a.warmup)))
            return
        import torch.distributed as dist
        out = bench_gpt.run_multi(a.gpus, a.steps, a.warmup)
        if out is not None:
            print(json.dumps(out), flush=True)
        if dist.is_initialized():
            dist.destroy_process_group()
        return
    if a.model == "resnet50" and a.gpus == 1 and world == 1:
        import bench_resnet
        print(json.dumps(bench_resnet.run(a.steps, a.warmup, not a.no_cpu_baseline)))
        return
    if a.gpus == 1 and world == 1:
        out = run_gpu_single(a.steps, a.warmup)
        if not a.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline()
        if not a.no_secondary:
            out["secondary"] = {"gnmt": secondary_gnmt_single(min(a.steps, 40), a.warmup)}
        print(json.dumps(out))
        return
    from bench_multi import run_gpu_multi     # pipeline / hybrid partitions over NVLink peer channels
    out = run_gpu_multi(a.gpus, a.steps, a.warmup, a.model)
    if out is not None:
        print(json.dumps(out), flush=True)
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
