"""Stage generator front end (pipedream_b200/stagegen.py) against the reference's generator
(optimizer/convert_graph_to_model.py): tests/golden/stagegen_golden.json holds two small partitioned graphs written
for this test, what the reference's generator made of them (its generated stage modules, described), their
parameters under seed 0 and their output on a seeded input.  The same comparison on the reference's own
vgg16 / resnet50 test graphs was made when the golden file was written (make_golden.py --only stagegen); the file
records its outcome."""
import json
import os

import pytest
import torch

from pipedream_b200 import partition, stagegen, stages

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "stagegen_golden.json")))


def canonical(desc):
    """Every assignment of a stage's dataflow numbered in order (`a = a + b` and `c = a + b` read the same)."""
    out = []
    for st in desc["stages"]:
        cur, flow = {}, []
        for stt in st["flow"]:
            if stt[1] == "none":                # `x = None`: where the statement stands does not matter
                cur[stt[0]] = "None"
                continue
            args = [cur[a] if isinstance(a, str) else a for a in stt[2:]]
            cur[stt[0]] = "v%d" % len(flow)
            flow.append([cur[stt[0]], stt[1]] + args)
        out.append({"modules": [[n, k, dict(sorted(kw.items()))] for n, k, kw in st["modules"]], "flow": flow,
                    "returns": [cur[r] for r in st["returns"]], "inputs": list(st["inputs"]), "outputs": list(st["outputs"])})
    return out


def checksum(t):
    t = t.detach().double().flatten()
    k = min(8, t.numel())
    idx = torch.tensor([(j * (t.numel() - 1)) // max(1, k - 1) for j in range(k)], dtype=torch.long)
    return {"sum": t.sum().item(), "abs_sum": t.abs().sum().item(), "sq_sum": (t * t).sum().item(), "samples": t[idx].tolist()}


@pytest.mark.parametrize("name", sorted(GOLD["graphs"]))
def test_description_equals_the_generators(name):
    g = GOLD["graphs"][name]
    mine = stagegen.describe(g["text"], g["arch"])
    assert canonical(mine) == canonical(g["description"])
    # names the runtime and checkpoints depend on
    for a, b in zip(mine["stages"], g["description"]["stages"]):
        assert [m[0] for m in a["modules"]] == [m[0] for m in b["modules"]]
        assert a["inputs"] == b["inputs"] and a["outputs"] == b["outputs"]


@pytest.mark.parametrize("name", sorted(k for k, v in GOLD["graphs"].items() if "output" in v))
def test_stages_built_from_the_description_match_the_generated_modules(name):
    g = GOLD["graphs"][name]
    pkg = stages.SpecPackage(stagegen.describe(g["text"], g["arch"]))
    torch.manual_seed(0)
    model = pkg.model(torch.nn.CrossEntropyLoss())
    got = {}
    for si, (m, _, _) in enumerate(model[:-1]):
        for k, v in m.state_dict().items():
            got["%d.%s" % (si, k)] = checksum(v)
    assert sorted(got) == sorted(g["state_dict"])
    for k, want in g["state_dict"].items():
        assert got[k]["samples"] == pytest.approx(want["samples"], rel=1e-6, abs=1e-7), k
        assert got[k]["sq_sum"] == pytest.approx(want["sq_sum"], rel=1e-6, abs=1e-9), k
    torch.manual_seed(1)
    vals = {"input0": torch.randn(*g["input_shape"])}
    for (m, ins, outs) in model[:-1]:
        m.eval()
        r = m(*[vals[i] for i in ins])
        vals.update(dict(zip(outs, r if isinstance(r, tuple) else (r,))))
    out = vals[model[-2][2][0]].detach().double().flatten()
    assert torch.allclose(out, torch.tensor(g["output"], dtype=torch.float64), rtol=1e-5, atol=1e-6)
    assert model[-1][1] == [model[-2][2][0]] and model[-1][2] == ["loss"]


def test_the_reference_graphs_were_checked_when_the_golden_file_was_written():
    rec = GOLD["checked_on_reference_graphs"]
    assert set(rec) == {"vgg16_partitioned.txt", "resnet50_partitioned.txt", "profiles/gnmt_large/graph.txt, cut into 4 stages",
                        "profiles/gnmt_large/graph.txt, partitioned by partition.plan_graph for 4 GPUs"}
    assert rec["profiles/gnmt_large/graph.txt, cut into 4 stages"]["stages"] == 4
    assert all(r["equal_to_generator_output"] for r in rec.values())
    assert rec["resnet50_partitioned.txt"]["stages"] == 4 and rec["vgg16_partitioned.txt"]["stages"] == 3


def test_graph_errors_and_configuration_maps():
    line = "%s -- %s -- forward_compute_time=1.000, backward_compute_time=1.000, activation_size=1.000, parameter_size=0.000 -- stage_id=0"
    with pytest.raises(ValueError, match="not supported"):
        stagegen.describe("\n".join([line % ("node1", "Input"), line % ("node2", "Transpose(0, 1)"), "\tnode1 -- node2"]), "x")
    with pytest.raises(ValueError, match="cycle"):
        stagegen.describe("\n".join([line % ("node1", "ReLU(inplace)"), line % ("node2", "ReLU(inplace)"),
                                     "\tnode1 -- node2", "\tnode2 -- node1"]), "x")
    with pytest.raises(ValueError, match="unknown node"):
        stagegen.Graph.parse("\n".join([line % ("node1", "Input"), "\tnode1 -- node9"]))
    assert stagegen.parse_module("Conv2d(3, 8, kernel_size=(3, 3), stride=(2, 2), bias=False)") == (
        "Conv2d", {"in_channels": 3, "out_channels": 8, "kernel_size": [3, 3], "stride": [2, 2], "padding": [0, 0], "bias": False})
    assert stagegen.parse_module("ReLU(inplace)") == ("ReLU", {"inplace": True})
    assert stagegen.configuration_maps(3) == {"module_to_stage_map": [0, 1, 2, 2],
                                              "stage_to_rank_map": {"0": [0], "1": [1], "2": [2]}}
    assert stagegen.configuration_maps(2, [3, 1]) == {"module_to_stage_map": [0, 1, 1],
                                                      "stage_to_rank_map": {"0": [0, 1, 2], "1": [3]}}
    # activation sizes of nodes with several outputs are written as a list
    g = stagegen.Graph.parse(line.replace("activation_size=1.000", "activation_size=[2.0; 3.0]") % ("node1", "Input"))
    assert g.nodes["node1"].activation == 5.0


@pytest.mark.parametrize("name", sorted(k for k, v in GOLD["graphs"].items() if "output" in v))
@pytest.mark.parametrize("gpus,straight", [(2, True), (3, True), (4, False)])
def test_partitioner_and_generator_compose(name, gpus, straight):
    """Profile graph -> partition.plan_graph -> stagegen.describe -> SpecPackage: the stages, run one after the other
    with the weights of the unpartitioned network (carried over by graph node), give its output."""
    import re
    g = GOLD["graphs"][name]
    flat = stagegen.Graph.parse(re.sub(r"stage_id=\d+", "stage_id=0", g["text"]))
    groups, times, params, acts, outs = stagegen.chain_layers(flat)
    assert sum(len(x) for x in groups) == len(flat.nodes)
    assert all(not flat.nodes[grp[-1]].desc.startswith("Size") for grp in groups)      # no integer crosses a cut
    t, plan, text = partition.plan_graph(flat, gpus, 1e9, straight=straight, cost="b200")
    assert sum(r for _, _, r in plan) == gpus and plan[0][0] == 0 and plan[-1][1] == len(groups)
    whole = stages.SpecPackage(stagegen.describe(stagegen.with_stages(flat, groups, [(0, len(groups), 1)]), g["arch"]))
    parts = stages.SpecPackage(stagegen.describe(text, g["arch"]))
    assert len(parts.description["stages"]) == len(plan)
    conf = stagegen.configuration_maps(len(plan), [r for _, _, r in plan])
    assert conf["stage_to_rank_map"][str(len(plan) - 1)][-1] == gpus - 1
    assert conf["module_to_stage_map"] == list(range(len(plan))) + [len(plan) - 1]
    torch.manual_seed(0)
    wm = whole.model(torch.nn.CrossEntropyLoss())
    pm = parts.model(torch.nn.CrossEntropyLoss())
    # weights by graph node
    src = {}
    for (m, _, _), st in zip(wm[:-1], whole.description["stages"]):
        for lname, node in st["nodes"].items():
            src[node] = getattr(m, lname).state_dict()
    for (m, _, _), st in zip(pm[:-1], parts.description["stages"]):
        for lname, node in st["nodes"].items():
            getattr(m, lname).load_state_dict(src[node])
    torch.manual_seed(1)
    x = torch.randn(*g["input_shape"])

    def run(model):
        vals = {"input0": x}
        for (m, ins, outs_) in model[:-1]:
            m.eval()
            r = m(*[vals[i] for i in ins])
            vals.update(dict(zip(outs_, r if isinstance(r, tuple) else (r,))))
        return vals[model[-2][2][0]]
    assert torch.allclose(run(pm), run(wm), rtol=1e-5, atol=1e-6)


def test_translation_stages_from_a_graph():
    """The translation model's node kinds (tuple items, initial hidden states that read as None, concatenation,
    modules with several inputs, the composite blocks): the description equals the generator's, the stages built from
    it have the generated modules' parameter names and shapes, and they run end to end on the CPU."""
    g = GOLD["graphs"]["translation"]
    desc = stagegen.describe(g["text"], g["arch"])
    assert canonical(desc) == canonical(g["description"])
    pkg = stages.SpecPackage(desc)
    torch.manual_seed(0)
    model = pkg.model(torch.nn.CrossEntropyLoss())
    shapes = {}
    for si, (m, _, _) in enumerate(model[:-1]):
        for k, v in m.state_dict().items():
            shapes["%d.%s" % (si, k)] = list(v.shape)
    assert shapes == g["state_dict_shapes"]
    assert [st["inputs"] for st in desc["stages"]] == [st["inputs"] for st in g["description"]["stages"]]
    T, B, V = 7, 3, 40
    gen = torch.Generator().manual_seed(2)
    src = torch.randint(4, V, (T, B), generator=gen)
    tgt = torch.randint(4, V, (T, B), generator=gen)
    vals = {"input0": src, "input1": torch.tensor([T, T - 1, T - 2]), "input2": tgt}
    for (m, ins, outs) in model[:-1]:
        m.eval()
        r = m(*[vals[i] for i in ins])
        vals.update(dict(zip(outs, r if isinstance(r, tuple) else (r,))))
    out = vals[model[-2][2][0]]
    assert tuple(out.shape) == (T, B, V) and torch.isfinite(out).all()


@pytest.mark.parametrize("gpus", [2, 3, 4])
def test_partitioner_on_the_translation_graph(gpus):
    """plan_graph on the translation graph: no cut sends a tuple, an integer or a None across, and the stages it
    yields run end to end."""
    import re
    g = GOLD["graphs"]["translation"]
    flat = stagegen.Graph.parse(re.sub(r"stage_id=\d+", "stage_id=0", g["text"]))
    groups, times, params, acts, outs = stagegen.chain_layers(flat)
    for grp in groups[:-1]:
        last = flat.nodes[grp[-1]]
        assert not last.desc.startswith(("LSTM", "RecurrentAttention", "Size")), last.desc
    t, plan, text = partition.plan_graph(stagegen.Graph.parse(re.sub(r"stage_id=\d+", "stage_id=0", g["text"])), gpus, 1e9,
                                         straight=True)
    assert len(plan) == gpus
    model = stages.SpecPackage(stagegen.describe(text, g["arch"])).model(torch.nn.CrossEntropyLoss())
    T, B, V = 6, 2, 40
    gen = torch.Generator().manual_seed(4)
    vals = {"input0": torch.randint(4, V, (T, B), generator=gen), "input1": torch.tensor([T, T - 2]),
            "input2": torch.randint(4, V, (T, B), generator=gen)}
    for (m, ins, outs_) in model[:-1]:
        m.eval()
        for i in ins:
            assert torch.is_tensor(vals[i]), i          # only tensors travel
        r = m(*[vals[i] for i in ins])
        vals.update(dict(zip(outs_, r if isinstance(r, tuple) else (r,))))
    assert tuple(vals[model[-2][2][0]].shape) == (T, B, V)


def test_a_module_chain_becomes_a_profile_graph_and_back():
    """chain_graph writes what the profiler would have written for a plain chain; planned, described and rebuilt, the
    stages compute what the chain computes."""
    torch.manual_seed(0)
    nn = torch.nn
    chain = [nn.Conv2d(3, 8, 3, padding=1), nn.ReLU(inplace=True), nn.MaxPool2d(2, 2), nn.Conv2d(8, 8, 3, padding=1, bias=False),
             nn.BatchNorm2d(8), nn.ReLU(), nn.AvgPool2d(4), nn.Flatten(), nn.Linear(8, 5), nn.Dropout(0.3), nn.Linear(5, 4)]
    times = [(1.0 + i, 2.0 + i) for i in range(len(chain))]
    outs = [100.0 * (i + 1) for i in range(len(chain))]
    text = stagegen.chain_graph(chain, times, None, outs)
    g = stagegen.Graph.parse(text)
    assert len(g.nodes) == len(chain) + 2                      # + Input, + the Size node of the flatten
    assert [n.stage for n in g.nodes.values()] == [None] * len(g.nodes)
    t, plan, ptext = partition.plan_graph(stagegen.Graph.parse(text), 3, 1e9, straight=True)
    assert len(plan) == 3 and t > 0
    model = stages.SpecPackage(stagegen.describe(ptext, "chain")).model(nn.CrossEntropyLoss())
    # weights: node k + 2 of the graph is layer k of the chain (the flatten took two node numbers)
    node_layer, k = {}, 2
    for i, m in enumerate(chain):
        if isinstance(m, nn.Flatten):
            k += 2
            continue
        node_layer["node%d" % k] = m
        k += 1
    for (m, _, _), st in zip(model[:-1], stagegen.describe(ptext, "chain")["stages"]):
        for lname, node in st["nodes"].items():
            getattr(m, lname).load_state_dict(node_layer[node].state_dict())
    x = torch.randn(2, 3, 8, 8)
    want = x
    for m in chain:
        m.eval()
        want = m(want)
    vals = {"input0": x}
    for (m, ins, outs_) in model[:-1]:
        m.eval()
        r = m(*[vals[i] for i in ins])
        vals.update(dict(zip(outs_, r if isinstance(r, tuple) else (r,))))
    assert torch.allclose(vals[model[-2][2][0]], want, rtol=1e-5, atol=1e-6)
