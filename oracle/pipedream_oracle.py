"""CPU restatement of the reference's pipeline-parallel training step.  TEST INFRASTRUCTURE.

This module is the checker for the CUDA implementation in pipedream_b200/: only tests/,
__graft_entry__.smoke() and the CPU-baseline legs of bench.py import it.  Nothing in the
product imports it and it imports nothing from the product.

Everything here follows the reference (msr-fiddle/pipedream, `pipedream` branch) and is
pinned against it: tests/golden/*.json were produced by running the reference itself
(tests/golden/make_golden.py) and tests/test_oracle.py checks this file against them.

All arithmetic is fp32 on the CPU with plain torch tensor operations.
"""
import collections
import copy

import numpy as np
import torch
import torch.nn as nn


# --------------------------------------------------------------------------- #
# stage / rank arithmetic          (reference: runtime/runtime.py:129-175)
# --------------------------------------------------------------------------- #
def stage_assignment(module_to_stage_map, stage_to_rank_map, stage_to_depth_map, rank):
    """Which stage a rank serves, its replica index, neighbours and warm-up depth."""
    stage_to_rank_map = {int(k): list(v) for k, v in stage_to_rank_map.items()}
    stages = sorted(set(module_to_stage_map))
    rank_to_stage = {r: s for s, rs in stage_to_rank_map.items() for r in rs}
    num_ranks = len(rank_to_stage)
    stage = rank_to_stage[rank]
    in_stage = stage_to_rank_map[stage]
    if stage_to_depth_map is not None:
        warmup = stage_to_depth_map[str(stage)]                       # runtime.py:166-168
    else:
        warmup = num_ranks - 1                                        # runtime.py:170-175
        for s in range(stage):
            warmup -= len(stage_to_rank_map[s])
        warmup //= len(in_stage)
    return {
        "stage": stage, "num_stages": len(stages), "num_ranks": num_ranks,
        "rank_in_stage": in_stage.index(rank), "num_ranks_in_stage": len(in_stage),
        "num_ranks_in_first_stage": len(stage_to_rank_map[0]),
        "ranks_in_previous_stage": stage_to_rank_map[stage - 1] if stage > 0 else [],
        "ranks_in_next_stage": stage_to_rank_map[stage + 1] if stage < len(stages) - 1 else [],
        "num_warmup_minibatches": warmup,
        "is_criterion": stage == len(stages) - 1,
        "modules": [m for m, s in enumerate(module_to_stage_map) if s == stage],
    }


def num_iterations(loader_size, a):
    """runtime/runtime.py:659-671."""
    if a["stage"] == 0:
        return loader_size
    total = loader_size * a["num_ranks_in_first_stage"]
    assert total % a["num_ranks_in_stage"] == 0
    return total // a["num_ranks_in_stage"]


def adjusted_learning_rate(base_lr, a):
    """runtime/runtime.py:673-680."""
    if a["stage"] == 0:
        return base_lr
    return float(base_lr) * float(a["num_ranks_in_stage"]) / float(a["num_ranks_in_first_stage"])


# --------------------------------------------------------------------------- #
# replica routing                  (reference: runtime/communication.py:456-521, 583-608)
# --------------------------------------------------------------------------- #
def messaging_rows(num_ranks_in_stage, num_ranks_in_previous_stage):
    rows = []
    for i in range(num_ranks_in_stage):
        idx, row = i, []
        while idx < num_ranks_in_previous_stage:
            row.append(idx)
            idx += num_ranks_in_stage
        if row:
            rows.append(row)
    return rows


class RoutingCursor:
    """One of the two cursors (forward-receive or backward-send) over the messaging schedule."""

    def __init__(self, rank_in_stage, rows):
        self.rows = rows
        self.row = rank_in_stage
        while self.rows and self.row >= len(self.rows):        # communication.py:484-487
            self.row -= 1
        self.col = 0

    def current(self):
        return self.rows[self.row][self.col]

    def advance(self):                                         # communication.py:501-521
        self.col += 1
        if self.col == len(self.rows[self.row]):
            self.col = 0
            self.row -= 1
            if self.row == -1:
                self.row = len(self.rows) - 1


def routing_sequences(a, n):
    """Replica indices used over n minibatches: (fwd_recv, bwd_send, fwd_send, bwd_recv)."""
    r_prev, r_next = len(a["ranks_in_previous_stage"]), len(a["ranks_in_next_stage"])
    fwd_recv, bwd_send, fwd_send, bwd_recv = [], [], [], []
    if r_prev > 0:
        rows = messaging_rows(a["num_ranks_in_stage"], r_prev)
        cf, cb = RoutingCursor(a["rank_in_stage"], rows), RoutingCursor(a["rank_in_stage"], rows)
        for _ in range(n):
            fwd_recv.append(cf.current())
            cf.advance()
            bwd_send.append(cb.current())
            cb.advance()
    if r_next > 0:
        for mb in range(n):
            fwd_send.append((mb + a["rank_in_stage"]) % r_next)        # communication.py:606-607
            bwd_recv.append((mb + a["rank_in_stage"]) % r_next)        # communication.py:586-587
    return fwd_recv, bwd_send, fwd_send, bwd_recv


# --------------------------------------------------------------------------- #
# weight stashing                  (reference: runtime/optimizer.py:19-164)
# --------------------------------------------------------------------------- #
class StashingOracle:
    """deque(maxlen=num_versions) of cloned parameter sets with version tags, plus explicit
    SGD (momentum, dampening, nesterov, L2) / Adam (L2, eps 1e-8) update formulas."""

    def __init__(self, name, modules, num_versions, lr, momentum=0.0, dampening=0.0, weight_decay=0.0,
                 nesterov=False, betas=(0.9, 0.999), eps=1e-8, macrobatch=False):
        self.name = name
        self.modules = modules
        if macrobatch:
            num_versions = min(2, num_versions)                 # optimizer.py:36-38
        self.num_versions = num_versions
        self.update_interval = num_versions if macrobatch else 1   # optimizer.py:49-52
        self.lr, self.momentum, self.dampening = lr, momentum, dampening
        self.weight_decay, self.nesterov, self.betas, self.eps = weight_decay, nesterov, betas, eps
        self.params = [p for m in modules for p in m.parameters()]
        self.latest_version = 0
        self.current_version = 0
        self.batch_counter = 0
        self.steps = 0
        self.state = [dict() for _ in self.params]
        self.queue = collections.deque(maxlen=num_versions)     # optimizer.py:58-62
        for _ in range(num_versions):
            self.queue.append(([p.detach().clone() for p in self.params], 0))

    def _load(self, entry):
        values, version = entry
        with torch.autograd._unsafe_preserve_version_counter(tuple(self.params)), torch.no_grad():
            for p, v in zip(self.params, values):
                p.copy_(v)
        self.current_version = version

    def load_old_params(self):                                  # optimizer.py:110-112
        if self.num_versions > 1:
            self._load(self.queue[0])

    def load_new_params(self):                                  # optimizer.py:114-116
        if self.num_versions > 1:
            self._load(self.queue[-1])

    def zero_grad(self):                                        # optimizer.py:118-120
        if self.batch_counter % self.update_interval == 0:
            for p in self.params:
                p.grad = None

    def step(self):                                             # optimizer.py:122-164
        if self.batch_counter % self.update_interval != self.update_interval - 1:
            self.batch_counter += 1
            return
        with torch.autograd._unsafe_preserve_version_counter(tuple(self.params)), torch.no_grad():
            self.steps += 1
            for p, st in zip(self.params, self.state):
                if p.grad is None:
                    continue
                g = p.grad / self.update_interval                # optimizer.py:147-149
                if self.name == "SGD":
                    d = g + self.weight_decay * p if self.weight_decay != 0 else g
                    if self.momentum != 0:
                        if "buf" not in st:
                            st["buf"] = d.clone()
                        else:
                            st["buf"] = self.momentum * st["buf"] + (1 - self.dampening) * d
                        d = d + self.momentum * st["buf"] if self.nesterov else st["buf"]
                    p.add_(d, alpha=-self.lr)
                elif self.name == "Adam":
                    b1, b2 = self.betas
                    if self.weight_decay != 0:
                        g = g + self.weight_decay * p
                    m = st.get("m", torch.zeros_like(p))
                    v = st.get("v", torch.zeros_like(p))
                    m = m + (g - m) * (1 - b1)
                    v = v * b2 + (1 - b2) * g * g
                    st["m"], st["v"] = m, v
                    bc1 = 1 - b1 ** self.steps
                    bc2 = 1 - b2 ** self.steps
                    denom = v.sqrt() / (bc2 ** 0.5) + self.eps
                    p.add_(m / denom, alpha=-(self.lr / bc1))
                else:
                    raise ValueError(self.name)
        self.latest_version += 1
        if self.num_versions > 1:                               # optimizer.py:157-159
            self.queue.append(([p.detach().clone() for p in self.params], self.latest_version))
        self.batch_counter += 1


def version_trace(num_warmup, n, macrobatch=False):
    """[event, minibatch, version] for one stage of the 1F1B loop
    (runtime/image_classification/main_with_runtime.py:359-421 around optimizer.py)."""
    num_versions = num_warmup + 1
    if macrobatch:
        num_versions = min(2, num_versions)
    interval = num_versions if macrobatch else 1
    versions = collections.deque([0] * num_versions, maxlen=num_versions)
    latest, counter, trace = 0, 0, []

    def fwd(i):
        trace.append(["F", i, latest])

    def bwd(i):
        nonlocal latest, counter
        trace.append(["B", i, versions[0] if num_versions > 1 else latest])
        if counter % interval == interval - 1:
            latest += 1
            if num_versions > 1:
                versions.append(latest)
        counter += 1
        trace.append(["S", i, latest])

    for i in range(num_warmup):
        fwd(i)
    for i in range(n - num_warmup):
        fwd(num_warmup + i)
        bwd(i)
    for i in range(num_warmup):
        bwd(n - num_warmup + i)
    return trace


# --------------------------------------------------------------------------- #
# stage modules                    (reference: runtime/image_classification/models/vgg16/gpus=*/stage*.py)
# --------------------------------------------------------------------------- #
class OracleStage(nn.Module):
    """A chain of torch.nn layers named layer<N> as in the generated stage files."""

    def __init__(self, spec, first_id):
        super().__init__()
        self.steps = []
        idx = first_id
        for item in spec:
            if item == "flatten":
                self.steps.append(None)
                idx += 2
                continue
            kind, args = item[0], item[1:]
            layer = {"conv": lambda a: nn.Conv2d(a[0], a[1], kernel_size=3, stride=1, padding=1),
                     "relu": lambda a: nn.ReLU(inplace=True),
                     "pool": lambda a: nn.MaxPool2d(kernel_size=2, stride=2),
                     "linear": lambda a: nn.Linear(a[0], a[1]),
                     "dropout": lambda a: nn.Dropout(p=a[0])}[kind](args)
            setattr(self, "layer%d" % idx, layer)
            self.steps.append("layer%d" % idx)
            idx += 1
        for m in self.modules():                                 # vgg16/gpus=8/stage0.py:34-45
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
                nn.init.constant_(m.bias, 0)
            elif isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0, 0.01)
                nn.init.constant_(m.bias, 0)

    def forward(self, x):
        out = x.clone()
        for s in self.steps:
            out = out.view(out.size(0), -1) if s is None else getattr(self, s)(out)
        return out


def vgg16_spec():
    spec, cin = [], 3
    for v in [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"]:
        if v == "M":
            spec.append(("pool",))
        else:
            spec += [("conv", cin, v), ("relu",)]
            cin = v
    spec.append("flatten")
    spec += [("linear", 25088, 4096), ("relu",), ("dropout", 0.5), ("linear", 4096, 4096), ("relu",),
             ("dropout", 0.5), ("linear", 4096, 1000)]
    return spec


def vgg16_stages(cut):
    """cut: None (one stage), "conv4_3" (gpus=8 split: stage 0 ends with conv4_3, stage 1 starts with
    its ReLU) or "flatten" (gpus=16 split: stage 1 holds the three Linear layers)."""
    spec = vgg16_spec()
    if cut is None:
        return [OracleStage(spec, 2)]
    if cut == "conv4_3":
        k = [i for i, s in enumerate(spec) if s != "flatten" and s[0] == "conv"][9] + 1
    elif cut == "flatten":
        k = spec.index("flatten") + 1
    else:
        raise ValueError(cut)
    return [OracleStage(spec[:k], 2), OracleStage(spec[k:], 1)]


def disable_dropout(module):
    for m in module.modules():
        if isinstance(m, nn.Dropout):
            m.p = 0.0


# --------------------------------------------------------------------------- #
# whole-pipeline simulation
# --------------------------------------------------------------------------- #
class PipelineOracle:
    """Every rank of a pipeline simulated in one process, in fp32 on the CPU.

    model: list of (module, [input names], [output names]) ending with the criterion, as a
    stage package's model() returns it.  Ranks of a replicated stage get deep copies of the
    stage's modules (the reference builds them with the same seed in every process) and
    average their gradients per step as DistributedDataParallel does (runtime.py:258-262).
    """

    def __init__(self, model, module_to_stage_map, stage_to_rank_map, stage_to_depth_map, opt_name, opt_args,
                 macrobatch=False, loss_fn=None):
        self.s2r = {int(k): list(v) for k, v in stage_to_rank_map.items()}
        self.world = sum(len(v) for v in self.s2r.values())
        self.ranks = []
        for rank in range(self.world):
            a = stage_assignment(module_to_stage_map, stage_to_rank_map, stage_to_depth_map, rank)
            entries = [model[m] for m in a["modules"]]
            if a["rank_in_stage"] > 0:
                entries = [(copy.deepcopy(mod), i, o) for (mod, i, o) in entries]
            trainable = [mod for (mod, _, _) in entries if any(True for _ in mod.parameters())]
            args = dict(opt_args)
            args["lr"] = adjusted_learning_rate(opt_args["lr"], a) if opt_args.get("scale_lr", False) else opt_args["lr"]
            args.pop("scale_lr", None)
            opt = StashingOracle(opt_name, trainable, a["num_warmup_minibatches"] + 1, macrobatch=macrobatch, **args)
            self.ranks.append({"a": a, "entries": entries, "opt": opt, "stash": collections.deque(), "fwd_id": 0,
                               "bwd_id": 0, "trace": [], "losses": [], "done_bwd": 0})
        self.mailbox = collections.defaultdict(collections.deque)
        self.model = model
        self.module_to_stage_map = module_to_stage_map
        self.all_names_in, self.all_names_out = {}, {}
        for s in set(module_to_stage_map):
            ins, outs = set(), set()
            for m, st in enumerate(module_to_stage_map):
                if st == s:
                    ins.update(model[m][1])
                    outs.update(model[m][2])
            self.all_names_in[s], self.all_names_out[s] = ins, outs

    # boundary tensors of a stage
    def _stage_inputs(self, s):
        return [n for n in sorted(self.all_names_in[s]) if n not in self.all_names_out[s]]

    def _stage_outputs(self, s):
        return [n for n in sorted(self.all_names_out[s]) if n not in self.all_names_in[s] and n != "loss"]

    def run(self, loaders, n_first_stage):
        """loaders[rank] for the ranks of stage 0: iterables of (input, target)."""
        R = self.ranks
        for k, st in enumerate(R):
            a = st["a"]
            st["n"] = num_iterations(n_first_stage, a)
            st["cursor_f"] = st["cursor_b"] = None
            if a["ranks_in_previous_stage"]:
                rows = messaging_rows(a["num_ranks_in_stage"], len(a["ranks_in_previous_stage"]))
                st["cursor_f"] = RoutingCursor(a["rank_in_stage"], rows)
                st["cursor_b"] = RoutingCursor(a["rank_in_stage"], rows)
            st["loader"] = iter(loaders[k]) if a["stage"] == 0 else None
            w, n = a["num_warmup_minibatches"], st["n"]
            prog = [("F", i) for i in range(w)]
            for i in range(n - w):
                prog += [("F", w + i), ("B", i), ("S", i)]
            for i in range(w):
                prog += [("B", n - w + i), ("S", n - w + i)]
            st["prog"], st["pc"] = prog, 0
        progress = True
        while progress:
            progress = False
            for k, st in enumerate(R):
                while st["pc"] < len(st["prog"]):
                    kind, i = st["prog"][st["pc"]]
                    ok = {"F": self._forward, "B": self._backward, "S": self._step}[kind](k, i)
                    if not ok:
                        break
                    st["pc"] += 1
                    progress = True
        assert all(st["pc"] == len(st["prog"]) for st in R), "oracle pipeline deadlocked"

    def _forward(self, k, i):
        st = self.ranks[k]
        a = st["a"]
        s = a["stage"]
        tensors = {}
        if s == 0:
            x, y = next(st["loader"])
            tensors["input0"], tensors["target"] = x, y
        else:
            src = a["ranks_in_previous_stage"][st["cursor_f"].current()]
            names = self._stage_inputs(s) + ["target"]
            if any(not self.mailbox[(src, k, n, False)] for n in names):
                return False
            for n in names:
                t = self.mailbox[(src, k, n, False)].popleft()
                tensors[n] = t.requires_grad_() if t.is_floating_point() else t
            st["cursor_f"].advance()
        st["trace"].append(["F", i, st["opt"].latest_version])
        for (mod, ins, outs) in st["entries"]:
            if outs == ["loss"]:
                tensors["loss"] = mod(tensors[ins[0]], tensors["target"])
            else:
                o = mod(*[tensors[n] for n in ins])
                o = o if isinstance(o, tuple) else (o,)
                for n, t in zip(outs, o):
                    tensors[n] = t
        if a["is_criterion"]:
            st["losses"].append(float(tensors["loss"].detach()))
        else:
            dst = a["ranks_in_next_stage"][(st["fwd_id"] + a["rank_in_stage"]) % len(a["ranks_in_next_stage"])]
            for n in self._stage_outputs(s) + ["target"]:
                self.mailbox[(k, dst, n, False)].append(tensors[n].detach().clone())
        st["stash"].append(tensors)
        st["fwd_id"] += 1
        return True

    def _backward(self, k, i):
        st = self.ranks[k]
        a = st["a"]
        s = a["stage"]
        grads = {}
        if not a["is_criterion"]:
            src = a["ranks_in_next_stage"][(st["bwd_id"] + a["rank_in_stage"]) % len(a["ranks_in_next_stage"])]
            names = self._stage_outputs(s)
            if any(not self.mailbox[(src, k, n, True)] for n in names):
                return False
            for n in names:
                grads[n] = self.mailbox[(src, k, n, True)].popleft()
        opt = st["opt"]
        opt.zero_grad()
        opt.load_old_params()
        st["trace"].append(["B", i, opt.current_version if opt.num_versions > 1 else opt.latest_version])
        tensors = st["stash"].popleft()
        if a["is_criterion"]:
            outs, gts = [tensors["loss"]], [None]
        else:
            outs = [tensors[n] for n in self._stage_outputs(s)]
            gts = [grads[n] for n in self._stage_outputs(s)]
        in_names = [n for n in self._stage_inputs(s) if tensors[n].requires_grad]
        for n in in_names:
            tensors[n].retain_grad()
        torch.autograd.backward(tuple(outs), grad_tensors=tuple(gts))
        if s > 0:
            dst = a["ranks_in_previous_stage"][st["cursor_b"].current()]
            for n in in_names:
                self.mailbox[(k, dst, n, True)].append(tensors[n].grad.detach().clone())
            st["cursor_b"].advance()
        opt.load_new_params()
        st["bwd_id"] += 1
        st["done_bwd"] += 1
        return True

    def _step(self, k, i):
        st = self.ranks[k]
        a = st["a"]
        peers = self.s2r[a["stage"]]
        if len(peers) > 1:
            # replicas step together on averaged gradients
            if any(self.ranks[p]["done_bwd"] <= i for p in peers):
                return False
            if a["rank_in_stage"] == 0 and not st.get("averaged_%d" % i):
                lists = [self.ranks[p]["opt"].params for p in peers]
                for group in zip(*lists):
                    gs = [p.grad for p in group if p.grad is not None]
                    if gs:
                        avg = sum(gs) / len(peers)
                        for p in group:
                            p.grad = avg.clone()
                for p in peers:
                    self.ranks[p]["averaged_%d" % i] = True
            if not st.get("averaged_%d" % i):
                return False
        st["opt"].step()
        st["trace"].append(["S", i, st["opt"].latest_version])
        return True


# --------------------------------------------------------------------------- #
# sequence utilities and criteria (numpy / python loops, small cases)
# --------------------------------------------------------------------------- #
def revert_varlen(x, lengths):
    """out[t,b] = x[len[b]-1-t, b] for t < len[b], else 0
    (runtime/translation/seq2seq/csrc/pack_utils_kernel.cu:7-13,37-51)."""
    x = np.asarray(x)
    out = np.zeros_like(x)
    for b, L in enumerate(lengths):
        for t in range(int(L)):
            out[t, b] = x[int(L) - 1 - t, b]
    return out


def set_mask(lengths):
    """uint8 [T,B] with T = lengths[0]; 1 where t < len[b]
    (runtime/translation/seq2seq/csrc/pack_utils.cpp:13-31)."""
    T = int(lengths[0])
    out = np.zeros((T, len(lengths)), dtype=np.uint8)
    for t in range(T):
        for b, L in enumerate(lengths):
            out[t, b] = 1 if L > t else 0
    return out


def label_smoothing_loss(logits, target, padding_idx, smoothing, batch_size):
    """runtime/translation/seq2seq/train/smoothing.py:23-34 on [rows, V] logits (float64 numpy)."""
    x = np.asarray(logits, dtype=np.float64)
    mx = x.max(axis=1, keepdims=True)
    logp = x - mx - np.log(np.exp(x - mx).sum(axis=1, keepdims=True))
    total = 0.0
    for r, t in enumerate(target):
        if t == padding_idx:
            continue
        total += (1.0 - smoothing) * (-logp[r, t]) + smoothing * (-logp[r].mean())
    return total / batch_size


def cross_entropy_loss(logits, target):
    """torch.nn.CrossEntropyLoss() (mean) as used at runtime/image_classification/main_with_runtime.py:126."""
    x = np.asarray(logits, dtype=np.float64)
    mx = x.max(axis=1, keepdims=True)
    logp = x - mx - np.log(np.exp(x - mx).sum(axis=1, keepdims=True))
    return float(-np.mean([logp[r, t] for r, t in enumerate(target)]))


# --------------------------------------------------------------------------- #
# LSTM layer and additive attention as explicit tensor arithmetic
# --------------------------------------------------------------------------- #
def lstm_layer(x, w_ih, w_hh, b_ih, b_hh):
    """torch.nn.LSTM(I, H) forward (one layer, one direction, zero initial state, gate order i,f,g,o)
    written out step by step; x: [T,B,I].  What the translation stages run through cuDNN in the
    reference (runtime/translation/models/gnmt_large/gpus=4/stage0.py:11-19)."""
    T, B, _ = x.shape
    H = w_hh.shape[1]
    h = x.new_zeros(B, H)
    c = x.new_zeros(B, H)
    ys = []
    for t in range(T):
        gates = x[t] @ w_ih.t() + b_ih + h @ w_hh.t() + b_hh
        i, f, g, o = gates.split(H, dim=1)
        i, f, g, o = torch.sigmoid(i), torch.sigmoid(f), torch.tanh(g), torch.sigmoid(o)
        c = f * c + i * g
        h = o * torch.tanh(c)
        ys.append(h)
    return torch.stack(ys, 0)


def bahdanau_scores(pq, pk, linear_att, normalize_scalar, normalize_bias):
    """Normalised additive attention scores (runtime/translation/seq2seq/models/attention.py:84-114):
    pq [b,tq,n], pk [b,tk,n] -> [b,tq,tk]."""
    v = linear_att / linear_att.norm() * normalize_scalar
    s = torch.tanh(pq.unsqueeze(2) + pk.unsqueeze(1) + normalize_bias)
    return (s * v).sum(-1)
