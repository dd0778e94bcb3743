"""Stage generator front end: a partitioned profile graph (text) -> stage descriptions for `stages.SpecStage`.

The reference turns the partitioner's output - the profile graph with a `stage_id` on every node - into Python
source, one `stageN.py` per stage plus an `__init__.py` that lists `(StageN(), [inputs], [outputs])`
(optimizer/convert_graph_to_model.py:89-356 for a stage, :358-425 for the package, graph/graph.py:463-480 and
:644-660 for the text format).  Here the same graph becomes data: the declarations and the dataflow of every
stage in the form `SpecStage` executes (and `layers.nativize` then plans as a whole), so no source is written,
imported or kept in sync.  What has to agree with the reference's generator, and is checked against its output in
the tests, are the names: modules are `layer<k>` with k counting the stage's inputs first and then its nodes in the
generator's topological order, boundary tensors are `out<k>` counted over the stages in order, and the inputs and
outputs of a stage are listed in the string order of their node ids - the parameter names of a checkpoint and the
tensor names of the runtime's configuration follow from these.

Graph text: one line per node, `id -- description -- forward_compute_time=..., backward_compute_time=...,
activation_size=..., parameter_size=... -- stage_id=k`, then one line per edge, a tab followed by `src -- dst`.
"""
import ast
import collections

Node = collections.namedtuple("Node", "id desc fwd bwd activation parameters stage")

# positional parameters of the layer types a description may declare (torch.nn signatures)
_POSITIONAL = {
    "Conv2d": ["in_channels", "out_channels", "kernel_size", "stride", "padding", "dilation", "groups", "bias"],
    "BatchNorm2d": ["num_features", "eps", "momentum", "affine", "track_running_stats"],
    "ReLU": ["inplace"],
    "MaxPool2d": ["kernel_size", "stride", "padding", "dilation", "return_indices", "ceil_mode"],
    "AvgPool2d": ["kernel_size", "stride", "padding", "ceil_mode", "count_include_pad"],
    "Linear": ["in_features", "out_features", "bias"],
    "Dropout": ["p", "inplace"],
    "Embedding": ["num_embeddings", "embedding_dim", "padding_idx"],
    "LSTM": ["input_size", "hidden_size", "num_layers", "bias", "batch_first", "dropout", "bidirectional"],
}
# node kinds that are dataflow, not modules (convert_graph_to_model.py:14-25); of those, products, transposes and the
# speech model's sequence-length helper have no counterpart in SpecStage and are refused
_DATAFLOW = ("Input", "Size", "View", "Add", "hidden", "__getitem__", "Concat")
_UNSUPPORTED = ("Mul", "Transpose", "self.get_seq_lens", "MaskConv", "ResizeInput", "InferenceBatchSoftmax", "BatchRNN",
                "SequenceWise")


class Graph:
    """Nodes in file order, successor and predecessor lists in the order the edges appear in the file."""

    def __init__(self):
        self.nodes = collections.OrderedDict()
        self.succ = collections.OrderedDict()
        self.pred = collections.OrderedDict()

    @staticmethod
    def parse(text):
        g = Graph()
        for line in text.strip().split("\n"):
            if not line.startswith("\t"):
                parts = line.strip().split(" -- ")
                if len(parts) < 3:
                    raise ValueError("not a node line: %r" % line)
                meta = dict(kv.split("=", 1) for kv in parts[2].split(", "))
                act = meta["activation_size"]
                act = sum(float(x) for x in act.strip("[]").split("; ")) if "[" in act else float(act)
                stage = int(parts[3].split("=")[1]) if len(parts) > 3 and parts[3].strip() else None
                g.nodes[parts[0]] = Node(parts[0], parts[1], float(meta["forward_compute_time"]),
                                         float(meta["backward_compute_time"]), act, float(meta["parameter_size"]), stage)
            else:
                src, dst = line.strip().split(" -- ")
                g.succ.setdefault(src, []).append(dst)
                g.pred.setdefault(dst, []).append(src)
        for src, dsts in g.succ.items():
            for n in [src] + dsts:
                if n not in g.nodes:
                    raise ValueError("edge names an unknown node %r" % n)
        return g

    def drop_unused_items(self):
        """Sinks that only pick an item out of a tuple nobody reads are dropped before anything is generated
        (convert_graph_to_model.py:452-456, one sweep over the sinks of the graph as read)."""
        for nid in [n.id for n in self.nodes.values() if not self.succ.get(n.id) and n.desc.startswith("__getitem__")]:
            for p in self.pred.pop(nid, []):
                self.succ[p].remove(nid)
            self.succ.pop(nid, None)
            del self.nodes[nid]
        return self

    def stage_ids(self):
        return sorted({n.stage for n in self.nodes.values()}, key=lambda s: (s is None, s))

    def stage_nodes(self, stage):
        """The stage's nodes in the order the reference's sub-graph holds them (graph/graph.py:128-137 with
        add_edge, :70-81): file order, except that a node pulls its successors inside the stage in right behind
        it.  Input / output numbering and the ties of the topological order all follow this order."""
        seen = collections.OrderedDict()
        for n in self.nodes.values():
            if n.stage != stage:
                continue
            seen.setdefault(n.id, n)
            for s in self.succ.get(n.id, []):
                if self.nodes[s].stage == stage:
                    seen.setdefault(s, self.nodes[s])
        return list(seen.values())

    def order(self, stage):
        """The generator's order of a stage's nodes (graph/graph.py:291-317): a depth-first walk over the edges
        inside the stage, roots taken in the order of their descriptions and successors likewise, every node
        placed in front of the list when its walk ends.  Ties keep file order (the reference's sort is stable)."""
        inside = {n.id for n in self.stage_nodes(stage)}
        done, out = set(), []
        roots = sorted(self.stage_nodes(stage), key=lambda n: n.desc)
        for root in roots:
            if root.id in done:
                continue
            # iterative walk: (node, iterator over its sorted successors)
            stack = [(root.id, iter(self._sorted_succ(root.id, inside)))]
            active = {root.id}
            while stack:
                nid, it = stack[-1]
                nxt = next(it, None)
                if nxt is None:
                    stack.pop()
                    active.discard(nid)
                    done.add(nid)
                    out.insert(0, nid)
                elif nxt in active:
                    raise ValueError("the graph has a cycle through %s" % nxt)
                elif nxt not in done:
                    active.add(nxt)
                    stack.append((nxt, iter(self._sorted_succ(nxt, inside))))
        return [self.nodes[i] for i in out]

    def _sorted_succ(self, nid, inside):
        return sorted((s for s in self.succ.get(nid, []) if s in inside), key=lambda s: self.nodes[s].desc)


def chain_layers(g):
    """The graph as the chain of layers `partition.plan` cuts (the reference's partitioner walks antichains of the
    general graph, optimizer/optimizer_graph_hierarchical.py:200-260; the networks this runtime executes from
    descriptions are chains with short side branches, for which a topological order and its prefixes are enough).
    A position is a legal cut when every edge that crosses it carries a tensor - not the integer of a `Size` node and
    not the tuple of a recurrent layer whose items are picked apart by `__getitem__` nodes, neither of which can travel
    between stages (initial hidden states can: they read as None on either side) - and the nodes between two legal
    cuts form one layer.

    Returns (groups, times, param_bytes, act_bytes, out_bytes): groups[i] = node ids of layer i in execution order;
    times in seconds per minibatch (forward + backward, the graph records milliseconds); out_bytes[i] = bytes that
    cross a cut placed after layer i."""
    if len(g.stage_ids()) != 1:
        raise ValueError("chain_layers takes an unpartitioned graph (one stage id, or none)")
    g.drop_unused_items()
    order = [n.id for n in g.order(g.stage_ids()[0])]

    def of_hidden(nid):
        return g.nodes[nid].desc.startswith("__getitem__") and any(g.nodes[p].desc.startswith("hidden") for p in g.pred.get(nid, []))
    # items of the initial hidden state (None) cost nothing and depend on nothing: each goes right in front of its
    # reader, so that the one cut that would send a None across is the only one they forbid
    moved = [nid for nid in order if of_hidden(nid)]
    order = [nid for nid in order if nid not in moved]
    for nid in moved:
        readers = [order.index(v) for v in g.succ.get(nid, []) if v in order]
        order.insert(min(readers) if readers else len(order), nid)
    pos = {nid: i for i, nid in enumerate(order)}
    L = len(order)
    crossing = [set() for _ in range(L)]               # crossing[k]: sources of the edges over the cut after position k
    for u, vs in g.succ.items():
        for v in vs:
            for k in range(pos[u], pos[v]):
                crossing[k].add(u)
    def carries_tensor(u):
        if g.nodes[u].desc.startswith("Size") or of_hidden(u):
            return False
        succs = g.succ.get(u, [])
        return not (succs and all(g.nodes[v].desc.startswith("__getitem__") for v in succs)) or g.nodes[u].desc.startswith("hidden")
    groups, cur = [], []
    for k, nid in enumerate(order):
        cur.append(nid)
        legal = k == L - 1 or all(carries_tensor(u) for u in crossing[k])
        if legal:
            groups.append(cur)
            cur = []
    times = [sum(g.nodes[i].fwd + g.nodes[i].bwd for i in grp) * 1e-3 for grp in groups]
    params = [sum(g.nodes[i].parameters for i in grp) for grp in groups]
    acts = [sum(g.nodes[i].activation for i in grp) for grp in groups]
    outs = [sum(g.nodes[u].activation for u in crossing[pos[grp[-1]]]) if grp[-1] != order[-1] else 0.0 for grp in groups]
    return groups, times, params, acts, outs


def with_stages(g, groups, stages):
    """The text of `g` with a stage id on every node: layers stages[s] = (first, one past last, replicas) of `groups`
    (what `partition.plan` returns) become stage s.  The result is what `describe` takes."""
    stage_of = {}
    for s, (start, end, _) in enumerate(stages):
        for grp in groups[start:end]:
            for nid in grp:
                stage_of[nid] = s
    if len(stage_of) != len(g.nodes):
        raise ValueError("the stages do not cover every layer")
    lines = ["%s -- %s -- forward_compute_time=%.3f, backward_compute_time=%.3f, activation_size=%.3f, "
             "parameter_size=%.3f -- stage_id=%d" % (n.id, n.desc, n.fwd, n.bwd, n.activation, n.parameters, stage_of[n.id])
             for n in g.nodes.values()]
    for dst, srcs in g.pred.items():
        for src in srcs:
            lines.append("\t%s -- %s" % (src, dst))
    return "\n".join(lines)


def chain_graph(modules, times=None, param_bytes=None, out_bytes=None):
    """Profile-graph text of a plain chain of torch.nn layers (an `nn.Sequential`-like list): an `Input` node, one node
    per layer described by its repr (the profiler's form, `Conv2d(3, 64, kernel_size=(3, 3), ...)`), edges from each
    node to the next; a `torch.nn.Flatten` becomes the `Size(0)` / `View(-1)` pair the reference's traces hold.  times:
    per-layer (forward, backward) milliseconds; sizes in bytes - what `partition.measure_layer_times` measures; zeros
    when not given.  The result is what `partition.plan_graph` and, once partitioned, `describe` take."""
    import torch.nn as nn
    nodes, edges = [("node1", "Input", 0.0, 0.0, 0.0, 0.0)], []
    prev, k = "node1", 2
    for i, m in enumerate(modules):
        f, b = times[i] if times is not None else (0.0, 0.0)
        pb = float(param_bytes[i]) if param_bytes is not None else float(sum(p.numel() * p.element_size() for p in m.parameters()))
        ob = float(out_bytes[i]) if out_bytes is not None else 0.0
        if isinstance(m, nn.Flatten):
            size, view = "node%d" % k, "node%d" % (k + 1)
            nodes += [(size, "Size(0)", 0.0, 0.0, 4.0, 0.0), (view, "View(-1)", f, b, ob, 0.0)]
            edges += [(prev, size), (prev, view), (size, view)]
            prev, k = view, k + 2
            continue
        desc = repr(m).replace("\n", "")
        if isinstance(m, nn.ReLU) and m.inplace:
            desc = "ReLU(inplace)"
        kind = desc.split("(")[0]
        if kind not in _POSITIONAL:
            raise ValueError("layer %d (%s) is not a kind a stage description can hold" % (i, kind))
        nid = "node%d" % k
        nodes.append((nid, desc, f, b, ob, pb))
        edges.append((prev, nid))
        prev, k = nid, k + 1
    lines = ["%s -- %s -- forward_compute_time=%.3f, backward_compute_time=%.3f, activation_size=%.3f, parameter_size=%.3f"
             % n for n in nodes]
    return "\n".join(lines + ["\t%s -- %s" % e for e in edges])


def parse_module(desc):
    """`Conv2d(3, 64, kernel_size=(3, 3), ...)` -> ("Conv2d", {keyword arguments}); a bare `inplace` means True
    (the profiler prints modules with their repr, convert_graph_to_model.py:120-121)."""
    import re
    # composite modules of the translation model: the profiler prints their whole repr, the generator keeps the sizes
    # (convert_graph_to_model.py:129-152).  RecurrentAttention is declared as (input, hidden, context) there and taken as
    # (input_size, context_size, hidden_size) by the class: the two are equal in every shipped model, and the
    # generator's order is kept.
    if desc.startswith("EmuBidirLSTM"):
        m = re.search(r"LSTM\((\d+), (\d+)", desc)
        return "EmuBidirLSTM", {"input_size": int(m.group(1)), "hidden_size": int(m.group(2))}
    if desc.startswith("RecurrentAttention"):
        m = re.search(r"LSTM\((\d+), (\d+)\)", desc)
        k = re.search(r"in_features=(\d+), out_features=(\d+)", desc)
        return "RecurrentAttention", {"input_size": int(m.group(1)), "context_size": int(m.group(2)),
                                      "hidden_size": int(k.group(1))}
    if desc.startswith("Classifier"):
        k = re.search(r"in_features=(\d+), out_features=(\d+)", desc)
        return "Classifier", {"in_features": int(k.group(1)), "out_features": int(k.group(2))}
    tree = ast.parse(desc.replace("inplace)", "inplace=True)").replace("(inplace,", "(inplace=True,"), mode="eval").body
    if not isinstance(tree, ast.Call) or not isinstance(tree.func, ast.Name):
        raise ValueError("not a module description: %r" % desc)
    kind = tree.func.id
    if kind not in _POSITIONAL:
        raise ValueError("module type %r is not supported by SpecStage" % kind)
    names = _POSITIONAL[kind]
    kw = {}
    for i, a in enumerate(tree.args):
        kw[names[i]] = ast.literal_eval(a)
    for k in tree.keywords:
        kw[k.arg] = ast.literal_eval(k.value)
    kw = {k: (list(v) if isinstance(v, tuple) else v) for k, v in kw.items()}
    # the arguments a repr leaves out when they have their default value, written out (a description then reads the
    # same whether it comes from a graph or from a live module)
    if kind == "Conv2d":
        for k, d in (("kernel_size", None), ("stride", 1), ("padding", 0)):
            v = kw.get(k, d)
            kw[k] = [v, v] if isinstance(v, int) else v
        kw.setdefault("bias", True)
    elif kind == "BatchNorm2d":
        for k, d in (("eps", 1e-5), ("momentum", 0.1), ("affine", True), ("track_running_stats", True)):
            kw.setdefault(k, d)
    elif kind == "ReLU":
        kw.setdefault("inplace", False)
    elif kind == "MaxPool2d":
        kw.setdefault("stride", kw["kernel_size"])
        for k, d in (("padding", 0), ("dilation", 1), ("ceil_mode", False)):
            kw.setdefault(k, d)
    elif kind == "AvgPool2d":
        kw.setdefault("stride", kw["kernel_size"])
        kw.setdefault("padding", 0)
    elif kind == "Linear":
        kw.setdefault("bias", True)
    elif kind == "Embedding":
        kw.setdefault("padding_idx", None)
    return kind, kw


def _stage_inputs(g, stage):
    """{predecessor node id: local name `input<k>`} of a stage, numbered in the order the generator meets them
    (stage nodes in file order, each node's predecessors in edge order; a predecessor met twice takes the later
    number: convert_graph_to_model.py:44-66)."""
    names, k = collections.OrderedDict(), 0
    for n in g.stage_nodes(stage):
        preds = g.pred.get(n.id, [])
        if preds:
            for p in preds:
                if g.nodes[p].stage != stage:
                    if g.nodes[p].desc.startswith("hidden"):
                        continue                      # initial hidden states are None on the other side as well
                    names[p] = "input%d" % k
                    k += 1
        elif n.desc.startswith("Input"):
            names[n.id] = "input%d" % k
            k += 1
    return names


def _stage_outputs(g, stage, counter):
    """{node id: package-wide name `out<k>`} of the stage's nodes that feed another stage (or nothing at all),
    numbered on from `counter` (convert_graph_to_model.py:68-87: once per outgoing edge that leaves the stage)."""
    names = collections.OrderedDict()
    for n in g.stage_nodes(stage):
        succs = g.succ.get(n.id, [])
        if succs:
            for s in succs:
                if g.nodes[s].stage != stage:
                    if n.desc.startswith("hidden"):
                        continue
                    names[n.id] = "out%d" % counter
                    counter += 1
        else:
            names[n.id] = "out%d" % counter
            counter += 1
    return names, counter


def _by_node_id(names):
    return [names[k] for k in sorted(names)]


def describe_stage(g, stage):
    """Declarations, dataflow and returned values of one stage, with the generator's names."""
    for n in g.stage_nodes(stage):
        if n.desc.startswith(_UNSUPPORTED):
            raise ValueError("node kind %r (%s) is not supported by SpecStage" % (n.desc, n.id))
    inputs = _stage_inputs(g, stage)
    value = {}                       # node id -> name of the value that holds its result
    flow, modules, node_of = [], [], {}
    local_inputs = _by_node_id(inputs)                    # the order of forward()'s arguments
    for pos, name in enumerate(local_inputs):
        flow.append([name, "input", pos])
    k = 0
    for nid, name in inputs.items():                      # every input is cloned first
        flow.append(["out%d" % k, "clone", name])
        value[nid] = "out%d" % k
        k += 1
    for n in g.order(stage):
        res = "out%d" % k
        value.setdefault(n.id, res)
        preds = g.pred.get(n.id, [])
        if n.desc.startswith("Input") and not preds:
            pass
        elif n.desc.startswith("Size"):
            if n.desc != "Size(0)" or len(preds) != 1:
                raise ValueError("only Size(0) of one tensor is supported, got %r" % n.desc)
            flow.append([res, "size0", value[preds[0]]])
        elif n.desc.startswith("View"):
            sizes = [p for p in preds if g.nodes[p].desc.startswith("Size")]
            data = [p for p in preds if not g.nodes[p].desc.startswith("Size")]
            if n.desc != "View(-1)" or len(sizes) != 1 or len(data) != 1:
                raise ValueError("only x.view(x.size(0), -1) is supported, got %r" % n.desc)
            flow.append([res, "flatten", value[data[0]], value[sizes[0]]])
        elif n.desc.startswith("hidden"):
            pass                                          # no statement; its items read as None
        elif n.desc.startswith("__getitem__"):
            if len(preds) != 1:
                raise ValueError("__getitem__ takes one operand (%s)" % n.id)
            idx = int(n.desc[len("__getitem__("):-1])
            if "hidden" in g.nodes[preds[0]].desc:
                flow.append([res, "none"])
            else:
                flow.append([res, "getitem", value[preds[0]], idx])
        elif n.desc.startswith("Concat"):
            flow.append([res, "cat", int(n.desc[len("Concat("):-1])] + [value[p] for p in preds])
        elif n.desc.startswith("Add"):
            if len(preds) != 2:
                raise ValueError("Add takes two operands (%s)" % n.id)
            a, b = preds
            if len(g.succ.get(a, [])) > 1:                # the operand with other readers is not overwritten
                a, b = b, a
            flow.append([value[a], "add", value[a], value[b]])
            value[n.id] = value[a]
        else:
            kind, kw = parse_module(n.desc)
            name = "layer%d" % k
            modules.append([name, kind, kw])
            node_of[name] = n.id
            flow.append([res, name] + [value[p] for p in preds])
        k += 1
    outputs, _ = _stage_outputs(g, stage, 0)
    returns = [value[nid] for nid in sorted(outputs)]
    # "nodes": which graph node a module came from (to carry weights from one partition of a graph to another)
    return {"modules": modules, "flow": flow, "returns": returns, "nodes": node_of}


def describe(text, arch):
    """The whole package: {"arch", "stages": [{"modules", "flow", "returns", "inputs", "outputs"}, ...]} with the
    package-wide tensor names the runtime's configuration uses ("input0", "out0", ...)."""
    g = Graph.parse(text) if isinstance(text, str) else text
    g.drop_unused_items()
    ids = g.stage_ids()
    if ids == [None]:
        ids = [None]
    glob = {}
    k = 0
    for n in g.nodes.values():                            # the package's own inputs
        if not g.pred.get(n.id) and n.desc.startswith("Input"):
            glob[n.id] = "input%d" % k
            k += 1
    stages, counter = [], 0
    for s in ids:
        st = describe_stage(g, s)
        # (the generator initialises the weights itself for these two targets only: convert_graph_to_model.py:447)
        st["init"] = "generator" if arch in ("vgg16", "resnet50") else "none"
        ins = _stage_inputs(g, s)
        outs, counter = _stage_outputs(g, s, counter)
        st["inputs"] = [glob[nid] for nid in sorted(ins)]
        glob.update(outs)
        st["outputs"] = [outs[nid] for nid in sorted(outs)]
        stages.append(st)
    return {"arch": arch, "stages": stages}


def configuration_maps(num_stages, stage_to_num_ranks=None):
    """`module_to_stage_map` / `stage_to_rank_map` of the generated `mp_conf.json` (one rank per stage) or, with
    replication factors, `hybrid_conf.json` (convert_graph_to_model.py:508-540); the criterion is the last
    module and shares the last stage."""
    m2s = list(range(num_stages)) + [num_stages - 1]
    if stage_to_num_ranks is None:
        return {"module_to_stage_map": m2s, "stage_to_rank_map": {str(i): [i] for i in range(num_stages)}}
    if len(stage_to_num_ranks) != num_stages:
        raise ValueError("one replication factor per stage")
    ranks, at = {}, 0
    for i, r in enumerate(stage_to_num_ranks):
        ranks[str(i)] = list(range(at, at + r))
        at += r
    return {"module_to_stage_map": m2s, "stage_to_rank_map": ranks}
