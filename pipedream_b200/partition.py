"""Pipeline partitioner: cuts a chain of layers into stages and chooses how often to replicate each stage.

Same dynamic programme as the reference's optimizer/optimizer_graph_hierarchical.py:17-101 (`compute_partitioning`)
and the same back-tracking as its `analyze_partitioning` (:103-196), restricted to what this runtime runs: one level
(one NVLink domain) and a chain of layers (every prefix of the layer list is a valid cut; VGG-16, GNMT and ResNet-50
at block granularity are chains).  Two cost models:

  cost="reference"  the reference's formulas, term for term (a replicated stage pays a ring all-reduce of
                    4 (m-1) P / (m B) seconds ON TOP of its compute time; boundary transfers count only when an
                    activation compression ratio is given, as 2 x bytes / B).  Used to check this
                    implementation against the reference's own results (tests/golden/partition_golden.json).
  cost="b200"       re-costed for this runtime: layer times are CUDA-event times of the native kernels
                    (`measure_layer_times`), the gradient all-reduce of a replicated stage is bucketed and overlaps
                    the backward pass (the stage costs max(compute / m, all-reduce), not their sum), boundary tensors
                    cross NVLink on side streams in both directions at once (bytes / B per direction, hidden
                    unless larger than the stage time), and B is the measured peer-copy rate.

`plan(...)` returns the stages as (first layer, one past the last layer, replicas); `hybrid_conf(...)` turns them
into the `module_to_stage_map` / `stage_to_rank_map` dictionaries the runtime takes (the content of the reference's
hybrid_conf.json, optimizer/convert_graph_to_model.py:508-543).
"""
import math


class _Chain:
    def __init__(self, times, param_bytes, act_bytes, out_bytes):
        n = len(times)
        assert len(param_bytes) == n and len(act_bytes) == n and len(out_bytes) == n
        self.n = n
        self.t = [0.0]
        self.p = [0.0]
        self.a = [0.0]
        for i in range(n):
            self.t.append(self.t[-1] + times[i])
            self.p.append(self.p[-1] + param_bytes[i])
            self.a.append(self.a[-1] + act_bytes[i])
        self.out = list(out_bytes)

    def span(self, i, j):
        """Sums over layers i..j inclusive: (time, parameter bytes, activation bytes)."""
        return self.t[j + 1] - self.t[i], self.p[j + 1] - self.p[i], self.a[j + 1] - self.a[i]


def _stage_time(cost, t, p, m, bandwidth, allreduce_bandwidth):
    """Time per minibatch of a stage of compute time t and parameter bytes p replicated m times."""
    if cost == "reference":
        return (t + (4.0 * (m - 1) * p) / (bandwidth * m)) / m
    reduce = 2.0 * (m - 1) * p / (m * allreduce_bandwidth) if m > 1 else 0.0      # ring: 2 (m-1)/m P bytes per GPU
    return max(t / m, reduce)


def plan(times, param_bytes, act_bytes, out_bytes, num_gpus, bandwidth, straight=False, cost="b200",
         compression_ratio=None, allreduce_bandwidth=None, memory_bytes=None):
    """Best split of layers 0..L-1 over `num_gpus`.  times in seconds per minibatch (forward + backward), sizes in
    bytes per minibatch, bandwidth in bytes/s.  Returns (bottleneck time, [(start, end, replicas), ...])."""
    if cost not in ("reference", "b200"):
        raise ValueError(cost)
    ch = _Chain(times, param_bytes, act_bytes, out_bytes)
    L, M = ch.n, num_gpus
    arb = allreduce_bandwidth or bandwidth
    count_transfers = cost == "b200" or compression_ratio is not None
    ratio = compression_ratio if compression_ratio is not None else 1.0
    # best[j][m]: (time, (k, m_rest) or None, replicas of the last stage) for layers 0..j on m+1 GPUs
    best = [[(None, None, None)] * M for _ in range(L)]
    for j in range(L):
        t, p, a = ch.span(0, j)
        for m in range(1 if straight else M):
            if memory_bytes is not None and math.ceil((M - (m + 1)) / (m + 1)) * (a + p) > memory_bytes:
                continue
            best[j][m] = (_stage_time(cost, t, p, m + 1, bandwidth, arb), None, m + 1)
    for m in range(1, M):
        for j in range(1, L):
            cur = best[j][m]
            for k in range(j):
                for mp in range(1, 2 if straight else m + 1):
                    t, p, a = ch.span(k + 1, j)
                    if memory_bytes is not None and (a + p) * math.ceil((M - (m + 1)) / mp) > memory_bytes:
                        continue
                    prev = best[k][m - mp][0]
                    if prev is None:
                        continue
                    total = max(prev, _stage_time(cost, t, p, mp, bandwidth, arb))
                    if count_transfers:
                        if cost == "reference":
                            total = max(total, 2.0 * ch.out[k] / (bandwidth * mp) / ratio)
                            if j < L - 1:
                                total = max(total, 2.0 * ch.out[j] / (bandwidth * mp) / ratio)
                        else:
                            total = max(total, ch.out[k] / (bandwidth * mp))
                            if j < L - 1:
                                total = max(total, ch.out[j] / (bandwidth * mp))
                    if cur[0] is None or cur[0] > total:
                        cur = (total, (k, m - mp), mp)
            best[j][m] = cur
    # back-track from all layers on all GPUs
    j, m = L - 1, M - 1
    stages = []
    while True:
        time, split, reps = best[j][m]
        if time is None:
            raise ValueError("no partition fits the constraints")
        if split is None:
            stages.append((0, j + 1, reps))
            break
        k, m_rest = split
        stages.append((k + 1, j + 1, reps))
        j, m = k, m_rest
    stages.reverse()
    return best[L - 1][M - 1][0], stages


def plan_graph(graph, num_gpus, bandwidth, **kw):
    """`plan` on a profile graph (`stagegen.Graph`, unpartitioned): returns (bottleneck time, stages, partitioned
    graph text) - the text is the graph with a `stage_id` on every node, i.e. what the reference's partitioner writes
    as `gpus=N.txt` and `stagegen.describe` turns into stages."""
    from . import stagegen
    groups, times, params, acts, outs = stagegen.chain_layers(graph)
    t, stages = plan(times, params, acts, outs, num_gpus, bandwidth, **kw)
    return t, stages, stagegen.with_stages(graph, groups, stages)


def hybrid_conf(stages, num_layers, criterion=True):
    """`module_to_stage_map` / `stage_to_rank_map` for a model list of `num_layers` entries (+ the criterion, which
    joins the last stage), ranks numbered stage by stage."""
    m2s = []
    for s, (start, end, _) in enumerate(stages):
        m2s.extend([s] * (end - start))
    assert len(m2s) == num_layers
    if criterion:
        m2s.append(len(stages) - 1)
    s2r, rank = {}, 0
    for s, (_, _, reps) in enumerate(stages):
        s2r[s] = list(range(rank, rank + reps))
        rank += reps
    return {"module_to_stage_map": m2s, "stage_to_rank_map": s2r, "stage_to_depth_map": None}


def measure_layer_times(modules, example_inputs, steps=5, warmup=2):
    """Forward + backward CUDA-event time (seconds) of every module of a chain on the current device, the
    parameter bytes, the bytes of everything a module keeps for its backward pass approximated by its output, and
    its output bytes.  modules: native (already swapped) modules; example_inputs: what the first one takes."""
    import torch
    times, params, acts, outs = [], [], [], []
    x = example_inputs
    for mod in modules:
        ins = [t.detach().requires_grad_(t.is_floating_point()) for t in (x if isinstance(x, (tuple, list)) else (x,))]
        best = None
        out = None
        for it in range(warmup + steps):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = mod(*ins)
            outs_ = out if isinstance(out, (tuple, list)) else (out,)
            grads = [torch.ones_like(o) for o in outs_ if o.requires_grad]
            torch.autograd.backward([o for o in outs_ if o.requires_grad], grads)
            e.record()
            torch.cuda.synchronize()
            if it >= warmup:
                ms = s.elapsed_time(e)
                best = ms if best is None else min(best, ms)
        outs_ = out if isinstance(out, (tuple, list)) else (out,)
        nbytes = sum(o.numel() * o.element_size() for o in outs_)
        times.append(best * 1e-3)
        params.append(sum(p.numel() * p.element_size() for p in mod.parameters()))
        acts.append(nbytes)
        outs.append(nbytes)
        x = tuple(o.detach() for o in outs_)
    return times, params, acts, outs
