"""Stage-module packages in the reference's generated format, built from an op list.

The reference ships one generated Python package per partitioning
(runtime/image_classification/models/vgg16/gpus=8/{stage0,stage1,__init__}.py).
Those files are not available where this library runs, so the same objects are
produced here from a table of operators: `vgg16("gpus=8")` returns an object
with `arch()`, `model(criterion)` and `full_model()`, whose stages are
`torch.nn.Module`s with the same attribute names (`layer<N>`), parameter
shapes, forward order (`input.clone()` first, flatten as `size(0)` + `view`)
and initialisation (kaiming-normal fan_out convolutions, N(0, 0.01) linears,
zero biases, drawn in module order) as the generated files, so state_dicts
interchange and a fixed seed yields the same initial weights.
"""
import torch
import torch.nn as nn

_VGG16_CFG = [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"]


def _vgg16_ops():
    ops, cin = [], 3
    for v in _VGG16_CFG:
        if v == "M":
            ops.append(("pool",))
        else:
            ops.append(("conv", cin, v))
            ops.append(("relu",))
            cin = v
    ops.append(("flatten",))
    ops += [("linear", 25088, 4096), ("relu",), ("dropout", 0.5),
            ("linear", 4096, 4096), ("relu",), ("dropout", 0.5), ("linear", 4096, 1000)]
    return ops


class SequentialStage(nn.Module):
    """One pipeline stage: a straight chain of operators named layer<N> by position."""

    def __init__(self, ops, first_id):
        super().__init__()
        self._plan = []
        idx = first_id
        for op in ops:
            kind = op[0]
            name = "layer%d" % idx
            if kind == "conv":
                setattr(self, name, nn.Conv2d(op[1], op[2], kernel_size=(3, 3), stride=(1, 1), padding=(1, 1)))
            elif kind == "relu":
                setattr(self, name, nn.ReLU(inplace=True))
            elif kind == "pool":
                setattr(self, name, nn.MaxPool2d(kernel_size=2, stride=2, padding=0, dilation=1, ceil_mode=False))
            elif kind == "linear":
                setattr(self, name, nn.Linear(in_features=op[1], out_features=op[2], bias=True))
            elif kind == "dropout":
                setattr(self, name, nn.Dropout(p=op[1]))
            elif kind == "flatten":
                self._plan.append(("flatten", None))
                idx += 2          # size(0) and view() each take a node id in the generated code
                continue
            else:
                raise ValueError(kind)
            self._plan.append(("module", name))
            idx += 1
        self._initialize_weights()

    def _initialize_weights(self):
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode='fan_out', nonlinearity='relu')
                if m.bias is not None:
                    nn.init.constant_(m.bias, 0)
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.constant_(m.weight, 1)
                nn.init.constant_(m.bias, 0)
            elif isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0, 0.01)
                nn.init.constant_(m.bias, 0)

    def forward(self, input0):
        out = input0.clone()
        for kind, name in self._plan:
            if kind == "flatten":
                out = out.view(out.size(0), -1)
            else:
                out = getattr(self, name)(out)
        return out


class StagePackage:
    """What `importlib.import_module(--module)` returns for a generated package."""

    def __init__(self, arch_name, stage_ops, conf):
        self._arch = arch_name
        self._stage_ops = stage_ops
        self.conf = conf          # default {"module_to_stage_map", "stage_to_rank_map"}

    def arch(self):
        return self._arch

    def stages(self):
        out = []
        for s, ops in enumerate(self._stage_ops):
            out.append(SequentialStage(ops, first_id=2 if s == 0 else 1))
        return out

    def model(self, criterion):
        stages = self.stages()
        names = ["input0"] + ["out%d" % i for i in range(len(stages))]
        m = [(st, [names[i]], [names[i + 1]]) for i, st in enumerate(stages)]
        m.append((criterion, [names[-1]], ["loss"]))
        return m

    def full_model(self):
        return nn.Sequential(*self.stages())


# Where each shipped VGG-16 partitioning cuts the operator chain (index of the first operator
# of the next stage).  gpus=8: after conv4_3, before its ReLU (gpus=8/stage0.py:31, stage1.py:10);
# gpus=16: after the flatten (gpus=16/stage0.py:76-78); gpus=2: after conv2_2's ReLU... the
# single-stage package keeps everything together.
def _cut_index(ops, which):
    convs = [i for i, op in enumerate(ops) if op[0] == "conv"]
    if which == "conv4_3":
        return convs[9] + 1
    if which == "flatten":
        return [i for i, op in enumerate(ops) if op[0] == "flatten"][0] + 1
    if which == "pool3":
        return [i for i, op in enumerate(ops) if op[0] == "pool"][2] + 1
    raise ValueError(which)


def vgg16(partition="gpus=1", stage_to_rank_map=None):
    """VGG-16 stage package.  partition: "gpus=1" (one stage), "gpus=8" (2 stages, cut after
    conv4_3), "gpus=16" (2 stages, cut after the flatten), "gpus=4" (2 stages, cut after pool3)."""
    ops = _vgg16_ops()
    cuts = {"gpus=1": [], "gpus=8": ["conv4_3"], "gpus=16": ["flatten"], "gpus=4": ["pool3"]}[partition]
    idx = [0] + [_cut_index(ops, c) for c in cuts] + [len(ops)]
    stage_ops = [ops[idx[i]:idx[i + 1]] for i in range(len(idx) - 1)]
    n = len(stage_ops)
    module_to_stage = list(range(n)) + [n - 1]
    if stage_to_rank_map is None:
        stage_to_rank_map = {s: [s] for s in range(n)}
    conf = {"module_to_stage_map": module_to_stage, "stage_to_rank_map": stage_to_rank_map}
    return StagePackage("vgg16", stage_ops, conf)


def hybrid_conf(num_stages, stage_to_num_ranks):
    """Contiguous rank assignment written by the reference's code generator for
    `--stage_to_num_ranks_map s:r,...` (optimizer/convert_graph_to_model.py:508-543)."""
    ranks, nxt = {}, 0
    for s in range(num_stages):
        r = stage_to_num_ranks.get(s, 1)
        ranks[s] = list(range(nxt, nxt + r))
        nxt += r
    return {"module_to_stage_map": list(range(num_stages)) + [num_stages - 1], "stage_to_rank_map": ranks}


class SyntheticImages:
    """Iterable of (images, labels): N(0,1) images, uniform labels, one generator seed per step
    (stands in for ImageNet, which is not available; shapes and value distributions only)."""

    def __init__(self, batch, steps, seed=1234, num_classes=1000, size=224, pin=False):
        self.batch, self.steps, self.seed = batch, steps, seed
        self.num_classes, self.size, self.pin = num_classes, size, pin

    def __len__(self):
        return self.steps

    def __iter__(self):
        for step in range(self.steps):
            g = torch.Generator().manual_seed(self.seed + step)
            x = torch.randn(self.batch, 3, self.size, self.size, generator=g)
            y = torch.randint(0, self.num_classes, (self.batch,), generator=g)
            if self.pin:
                x, y = x.pin_memory(), y.pin_memory()
            yield x, y


# --------------------------------------------------------------------------- #
# translation: the 8+8-layer GNMT ("gnmt_large"), 4-stage partitioning
# --------------------------------------------------------------------------- #
class GnmtPackage:
    """Stage package of runtime/translation/models/gnmt_large/gpus=4/__init__.py: four stages whose
    boundary tensors are named as there (out0, out1, out12, out13, out14, out15, out12again, out18)."""

    def __init__(self, hidden=1024, vocab=32320, dropout=0.2, stage_to_rank_map=None):
        self.hidden, self.vocab, self.dropout = hidden, vocab, dropout
        ranks = stage_to_rank_map or {s: [s] for s in range(4)}
        self.conf = {"module_to_stage_map": [0, 1, 2, 3, 3], "stage_to_rank_map": ranks}

    def arch(self):
        return "gnmt_large"

    def stages(self):
        from . import gnmt_blocks as gb
        h, v, p = self.hidden, self.vocab, self.dropout
        return [gb.GnmtStage0(h, v, p), gb.GnmtStage1(h, v, p), gb.GnmtStage2(h, p), gb.GnmtStage3(h, v, p)]

    def model(self, criterion):
        s = self.stages()
        return [
            (s[0], ["input0", "input1"], ["out0", "out1"]),
            (s[1], ["out0", "input1", "out1", "input2"], ["out12", "out13"]),
            (s[2], ["out12", "out13"], ["out14", "out15", "out12again"]),
            (s[3], ["out12again", "out14", "out15"], ["out18"]),
            (criterion, ["out18"], ["loss"]),
        ]

    def full_model(self):
        return torch.nn.ModuleList(self.stages())


def gnmt_large(hidden=1024, vocab=32320, dropout=0.2, stage_to_rank_map=None):
    return GnmtPackage(hidden, vocab, dropout, stage_to_rank_map)


class SyntheticTranslation:
    """Iterable of ((src, src_len), (tgt, tgt_len)) batches in the collate format of the reference's
    loader (runtime/translation/seq2seq/data/dataset.py:54-61): [T,B] int64 token matrices, BOS first,
    EOS last, PAD=0 beyond the length, batch sorted by source length (descending).  Lengths are uniform in
    [min_len, max_len]; token ids follow a Zipf(s=1.1) rank distribution mapped onto ids 4..vocab_used-1
    (stands in for WMT En-De, which is not available)."""

    PAD, UNK, BOS, EOS = 0, 1, 2, 3

    def __init__(self, batch, steps, seed=4321, min_len=20, max_len=50, vocab_used=32000, zipf_s=1.1):
        self.batch, self.steps, self.seed = batch, steps, seed
        self.min_len, self.max_len, self.vocab_used = min_len, max_len, vocab_used
        ranks = torch.arange(1, vocab_used - 4 + 1, dtype=torch.float64)
        self.weights = ranks.pow(-zipf_s)

    def __len__(self):
        return self.steps

    def _side(self, lengths, g):
        T, B = int(lengths.max()), len(lengths)
        ids = torch.multinomial(self.weights, T * B, replacement=True, generator=g).view(T, B) + 4
        out = torch.zeros(T, B, dtype=torch.int64)
        for b, L in enumerate(lengths.tolist()):
            out[:L, b] = ids[:L, b]
            out[0, b] = self.BOS
            out[L - 1, b] = self.EOS
        return out

    def __iter__(self):
        for step in range(self.steps):
            g = torch.Generator().manual_seed(self.seed + step)
            src_len = torch.randint(self.min_len, self.max_len + 1, (self.batch,), generator=g)
            tgt_len = torch.randint(self.min_len, self.max_len + 1, (self.batch,), generator=g)
            order = torch.argsort(src_len, descending=True, stable=True)
            src_len, tgt_len = src_len[order], tgt_len[order]
            yield (self._side(src_len, g), src_len.tolist()), (self._side(tgt_len, g), tgt_len.tolist())


# --------------------------------------------------------------------------- #
# ResNet-50 (v1.5: the stride of a bottleneck sits on its 3x3 convolution), straight pipeline
# --------------------------------------------------------------------------- #
class Bottleneck(nn.Module):
    """1x1 -> 3x3 (stride) -> 1x1 (x4) with BatchNorm after each convolution and a projection shortcut when
    the shape changes; the layer mix of runtime/image_classification/models/resnet50/gpus=4/stage*.py."""

    def __init__(self, cin, width, stride):
        super().__init__()
        cout = 4 * width
        self.conv1 = nn.Conv2d(cin, width, kernel_size=(1, 1), stride=(1, 1), bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.relu1 = nn.ReLU(inplace=True)
        self.conv2 = nn.Conv2d(width, width, kernel_size=(3, 3), stride=(stride, stride), padding=(1, 1), bias=False)
        self.bn2 = nn.BatchNorm2d(width)
        self.relu2 = nn.ReLU(inplace=True)
        self.conv3 = nn.Conv2d(width, cout, kernel_size=(1, 1), stride=(1, 1), bias=False)
        self.bn3 = nn.BatchNorm2d(cout)
        self.has_projection = stride != 1 or cin != cout
        if self.has_projection:
            self.down_conv = nn.Conv2d(cin, cout, kernel_size=(1, 1), stride=(stride, stride), bias=False)
            self.down_bn = nn.BatchNorm2d(cout)
        self.relu3 = nn.ReLU(inplace=True)

    def forward(self, x):
        out = self.relu1(self.bn1(self.conv1(x)))
        out = self.relu2(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        shortcut = self.down_bn(self.down_conv(x)) if self.has_projection else x
        return self.relu3(out + shortcut)


class ResNetStem(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = nn.Conv2d(3, 64, kernel_size=(7, 7), stride=(2, 2), padding=(3, 3), bias=False)
        self.bn = nn.BatchNorm2d(64)
        self.relu = nn.ReLU(inplace=True)
        self.pool = nn.MaxPool2d(kernel_size=3, stride=2, padding=1, dilation=1, ceil_mode=False)

    def forward(self, x):
        return self.pool(self.relu(self.bn(self.conv(x))))


class ResNetHead(nn.Module):
    def __init__(self, num_classes=1000):
        super().__init__()
        self.pool = nn.AvgPool2d(kernel_size=7, stride=1, padding=0)
        self.fc = nn.Linear(2048, num_classes)

    def forward(self, x):
        out = self.pool(x)
        return self.fc(out.view(out.size(0), -1))


class ResNetStage(nn.Module):
    def __init__(self, parts):
        super().__init__()
        self.parts = nn.ModuleList(parts)
        for m in self.modules():                      # resnet50/gpus=4/stage1.py:114-120
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode='fan_out', nonlinearity='relu')
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.constant_(m.weight, 1)
                nn.init.constant_(m.bias, 0)
            elif isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0, 0.01)
                nn.init.constant_(m.bias, 0)

    def forward(self, input0):
        out = input0.clone()
        for p in self.parts:
            out = p(out)
        return out


def _resnet50_units():
    """(kind, args, forward MACs per sample, output shape (C, H)) of the 18 cut units: stem, 16 blocks, head."""
    units = [("stem", (), 112 * 112 * 64 * 147, (64, 56))]
    cin, hw = 64, 56
    for width, blocks, stride in ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)):
        for b in range(blocks):
            st = stride if b == 0 else 1
            ho, cout = hw // st, 4 * width
            macs = hw * hw * cin * width + ho * ho * 9 * width * width + ho * ho * width * cout
            if st != 1 or cin != cout:
                macs += ho * ho * cin * cout
            units.append(("block", (cin, width, st), macs, (cout, ho)))
            cin, hw = cout, ho
    units.append(("head", (), 2048 * 1000, (1000, None)))
    return units


def _balanced_cuts(costs, k):
    """Split `costs` into k contiguous non-empty groups minimising the largest group sum (what the
    reference's partitioner optimises for a straight pipeline, optimizer_graph_hierarchical.py:20-100);
    returns the group sizes."""
    n = len(costs)
    pre = [0]
    for c in costs:
        pre.append(pre[-1] + c)
    INF = float("inf")
    best = [[INF] * (n + 1) for _ in range(k + 1)]
    arg = [[0] * (n + 1) for _ in range(k + 1)]
    best[0][0] = 0
    for j in range(1, k + 1):
        for i in range(j, n + 1):
            for m in range(j - 1, i):
                v = max(best[j - 1][m], pre[i] - pre[m])
                if v < best[j][i]:
                    best[j][i], arg[j][i] = v, m
    sizes, i = [], n
    for j in range(k, 0, -1):
        m = arg[j][i]
        sizes.append(i - m)
        i = m
    return sizes[::-1]


def resnet50(num_stages=1, stage_to_rank_map=None):
    """ResNet-50 cut at residual-block boundaries into `num_stages` (1..18) consecutive stages of balanced
    forward FLOPs; one tensor crosses each boundary.  (The reference's generated partitions cut inside
    blocks, so that the block input travels beside the main path, models/resnet50/gpus=4/__init__.py:13-18;
    cutting between blocks moves the same bytes once instead.)"""
    units = _resnet50_units()
    if not 1 <= num_stages <= len(units):
        raise ValueError("resnet50: 1..%d stages" % len(units))
    sizes = _balanced_cuts([u[2] for u in units], num_stages)
    chunks, i = [], 0
    for sz in sizes:
        chunks.append(units[i:i + sz])
        i += sz

    class _Pkg(StagePackage):
        def stages(self_inner):
            out = []
            for ch in chunks:
                parts = []
                for u in ch:
                    if u[0] == "stem":
                        parts.append(ResNetStem())
                    elif u[0] == "head":
                        parts.append(ResNetHead())
                    else:
                        parts.append(Bottleneck(*u[1]))
                out.append(ResNetStage(parts))
            return out

        def boundary_shapes(self_inner, batch):
            """{tensor name: shape} of the network input, every stage output and the target."""
            shapes = {"input0": (batch, 3, 224, 224), "target": (batch,)}
            for k, ch in enumerate(chunks):
                c, hw = ch[-1][3]
                shapes["out%d" % k] = (batch, c) if hw is None else (batch, c, hw, hw)
            return shapes

        def stage_macs(self_inner):
            return [sum(u[2] for u in ch) for ch in chunks]

    n = len(chunks)
    ranks = stage_to_rank_map or {s: [s] for s in range(n)}
    return _Pkg("resnet50", None, {"module_to_stage_map": list(range(n)) + [n - 1], "stage_to_rank_map": ranks})


def gpt2(num_stages=1, layers=24, hidden=1024, heads=16, seq_len=512, vocab=50257, dropout=0.1, stage_to_rank_map=None):
    """GPT-style decoder cut into `num_stages` consecutive stages: embeddings with the first blocks, final
    LayerNorm and the output projection with the last.  The vocabulary is padded to a multiple of 64 (50257 ->
    50304) so that logits rows are 16-byte aligned; the padding classes are never targets."""
    from . import gpt_blocks as gb
    vpad = (vocab + 63) // 64 * 64
    units = ["embed"] + ["block"] * layers + ["head"]
    costs = [1] + [12 * hidden * hidden + 2 * seq_len * hidden] * layers + [hidden * vpad]
    sizes = _balanced_cuts(costs, num_stages)
    chunks, i = [], 0
    for sz in sizes:
        chunks.append(units[i:i + sz])
        i += sz

    class _Pkg(StagePackage):
        def stages(self_inner):
            out = []
            for ch in chunks:
                parts = []
                for u in ch:
                    if u == "embed":
                        parts.append(gb.Embed(vpad, seq_len, hidden, dropout))
                    elif u == "head":
                        parts.append(gb.Head(hidden, vpad))
                    else:
                        parts.append(gb.Block(hidden, heads, dropout))
                out.append(gb.GptStage(parts))
            return out

        def boundary_shapes(self_inner, batch):
            shapes = {"input0": (batch, seq_len), "target": (batch * seq_len,)}
            for k, ch in enumerate(chunks):
                shapes["out%d" % k] = (batch * seq_len, vpad) if ch[-1] == "head" else (batch, seq_len, hidden)
            return shapes

    n = len(chunks)
    ranks = stage_to_rank_map or {s: [s] for s in range(n)}
    pkg = _Pkg("gpt2", None, {"module_to_stage_map": list(range(n)) + [n - 1], "stage_to_rank_map": ranks})
    pkg.vocab, pkg.vocab_padded, pkg.seq_len = vocab, vpad, seq_len
    return pkg


class SyntheticTokens:
    """Iterable of (tokens [B, T] int64, next-token targets [B*T] int64): ids uniform over the vocabulary."""

    def __init__(self, batch, steps, seq_len=512, vocab=50257, seed=2468):
        self.batch, self.steps, self.seq_len, self.vocab, self.seed = batch, steps, seq_len, vocab, seed

    def __len__(self):
        return self.steps

    def __iter__(self):
        for step in range(self.steps):
            g = torch.Generator().manual_seed(self.seed + step)
            ids = torch.randint(0, self.vocab, (self.batch, self.seq_len + 1), generator=g)
            yield ids[:, :-1].contiguous(), ids[:, 1:].contiguous().view(-1)


# --------------------------------------------------------------------------- #
# stages from a declarative description (the form a stage generator emits)
# --------------------------------------------------------------------------- #
class SpecStage(nn.Module):
    """A pipeline stage built from a description instead of a source file: the declarations
    `[name, type, kwargs]` in order, and the dataflow `[result, op, operands...]` with op one of a declared
    module's name, "input", "clone", "add", "size0", "flatten", "getitem", "none", "cat" - the statement kinds the reference's stage
    generator emits (optimizer/convert_graph_to_model.py:89-356 writes them as Python source, e.g.
    runtime/image_classification/models/resnet50/gpus=4/stage1.py:7-120).  Modules are created in declaration
    order and initialised as the generated files do (`kaiming_normal_(fan_out)` convolutions, unit BatchNorm),
    so under the same seed the parameters equal those of the generated stage, name for name."""

    TYPES = {"Conv2d": nn.Conv2d, "BatchNorm2d": nn.BatchNorm2d, "ReLU": nn.ReLU, "MaxPool2d": nn.MaxPool2d,
             "AvgPool2d": nn.AvgPool2d, "Linear": nn.Linear, "Dropout": nn.Dropout, "Embedding": nn.Embedding,
             "LSTM": nn.LSTM}

    @classmethod
    def module_type(cls, kind):
        """torch.nn layers, and the translation model's composite blocks (seq2seq/models/encoder.py:24-62,
        decoder.py:13-118 in the reference; restated in gnmt_blocks.py)."""
        if kind in cls.TYPES:
            return cls.TYPES[kind]
        if kind in ("EmuBidirLSTM", "RecurrentAttention", "Classifier"):
            from . import gnmt_blocks
            return getattr(gnmt_blocks, kind)
        raise ValueError("module type %r is not known to SpecStage" % kind)

    def __init__(self, spec):
        super().__init__()
        for name, kind, kwargs in spec["modules"]:
            kw = {k: (tuple(v) if isinstance(v, list) else v) for k, v in kwargs.items()}
            setattr(self, name, self.module_type(kind)(**kw))
        self._flow = [tuple(st) for st in spec["flow"]]
        self._returns = list(spec["returns"])
        # "init": "generator" = what the generator appends for its vgg16 / resnet50 targets
        # (optimizer/convert_graph_to_model.py:331-344: zero convolution biases and N(0, 0.01) Linear weights as well);
        # "none" = torch's defaults; otherwise the initialisation of the shipped resnet50 stage files
        init = spec.get("init", "shipped")
        for m in self.modules():
            if init == "none":
                break
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode='fan_out', nonlinearity='relu')
                if init == "generator" and m.bias is not None:
                    nn.init.constant_(m.bias, 0)
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.constant_(m.weight, 1)
                nn.init.constant_(m.bias, 0)
            elif init == "generator" and isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0, 0.01)
                nn.init.constant_(m.bias, 0)

    def forward(self, *inputs):
        v = {}
        for st in self._flow:
            res, op = st[0], st[1]
            if op == "input":
                v[res] = inputs[st[2]]
            elif op == "clone":
                v[res] = v[st[2]].clone()
            elif op == "add":
                v[res] = v[st[2]] + v[st[3]]
            elif op == "size0":
                v[res] = v[st[2]].size(0)
            elif op == "flatten":
                v[res] = v[st[2]].view(v[st[3]], -1)
            elif op == "getitem":
                v[res] = v[st[2]][st[3]]
            elif op == "none":
                v[res] = None
            elif op == "cat":
                v[res] = torch.cat([v[a] for a in st[3:]], st[2])
            else:
                v[res] = getattr(self, op)(*[v[a] for a in st[2:]])
        out = tuple(v[n] for n in self._returns)
        return out[0] if len(out) == 1 else out


class SpecPackage:
    """Stage package (`arch`, `model(criterion)`, `conf`) over SpecStage descriptions:
    {"arch": ..., "stages": [{"modules", "flow", "returns", "inputs", "outputs"}, ...]}."""

    def __init__(self, description):
        self.description = description
        n = len(description["stages"])
        self.conf = {"module_to_stage_map": list(range(n)) + [n - 1],
                     "stage_to_rank_map": {s: [s] for s in range(n)}, "stage_to_depth_map": None}

    def arch(self):
        return self.description["arch"]

    def model(self, criterion):
        out = [(SpecStage(st), list(st["inputs"]), list(st["outputs"])) for st in self.description["stages"]]
        out.append((criterion, [self.description["stages"][-1]["outputs"][0]], ["loss"]))
        return out
