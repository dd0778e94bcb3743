"""The CPU oracle (oracle/pipedream_oracle.py) against golden vectors recorded from the reference
(tests/golden/make_golden.py), and the product's host-side index logic against the same vectors."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import pipedream_oracle as oracle
from pipedream_b200 import communication, optimizer as pd_optimizer, runtime as pd_runtime, schedule, stages

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    with open(os.path.join(GOLD, name)) as f:
        return json.load(f)


ROUTING = load("routing_golden.json")
STASH = load("stashing_golden.json")


@pytest.mark.parametrize("cfg", sorted(ROUTING))
def test_stage_assignment_and_routing(cfg):
    g = ROUTING[cfg]
    s2r = {int(k): v for k, v in g["stage_to_rank_map"].items()}
    for rec in g["ranks"]:
        a = oracle.stage_assignment(g["module_to_stage_map"], s2r, g["stage_to_depth_map"], rec["rank"])
        b = pd_runtime.stage_assignment(len(g["module_to_stage_map"]),
                                        {"module_to_stage_map": g["module_to_stage_map"], "stage_to_rank_map": s2r,
                                         "stage_to_depth_map": g["stage_to_depth_map"]}, rec["rank"])
        for impl in (a, b):
            for key in ("stage", "rank_in_stage", "num_ranks_in_stage", "num_stages", "num_ranks",
                        "num_ranks_in_first_stage", "num_warmup_minibatches", "is_criterion",
                        "ranks_in_previous_stage", "ranks_in_next_stage"):
                assert impl[key] == rec[key], (cfg, rec["rank"], key)
        assert oracle.adjusted_learning_rate(0.1, a) == rec["adjusted_lr_0.1"]
        if rec["num_iterations_24"] is not None:
            assert oracle.num_iterations(24, a) == rec["num_iterations_24"]
        # oracle routing
        fr, bs, fs, br = oracle.routing_sequences(a, 24)
        assert (fr, bs, fs, br) == (rec["fwd_recv"], rec["bwd_send"], rec["fwd_send"], rec["bwd_recv"])
        # product routing
        if rec["ranks_in_previous_stage"]:
            ms = communication.MessagingSchedule(rec["rank_in_stage"], rec["num_ranks_in_stage"],
                                                 len(rec["ranks_in_previous_stage"]))
            assert ms.rows == rec["messaging_schedule"]
            got_f, got_b = [], []
            for _ in range(24):
                got_f.append(ms.index(False)); ms.increment(False)
                got_b.append(ms.index(True)); ms.increment(True)
            assert got_f == rec["fwd_recv"] and got_b == rec["bwd_send"]
        if rec["ranks_in_next_stage"]:
            n_next = len(rec["ranks_in_next_stage"])
            assert [communication.forward_send_index(m, rec["rank_in_stage"], n_next) for m in range(24)] == rec["fwd_send"]
            assert [communication.backward_recv_index(m, rec["rank_in_stage"], n_next) for m in range(24)] == rec["bwd_recv"]


def test_truth_table():
    """Weight-stashing known-answer test of the reference (runtime/tests/backprop/sgd_with_stashing.py)."""
    expect = {"1": (False, False), "2": (True, False), "3": (True, True)}
    for k, rec in STASH["truth_table"].items():
        assert (rec["equal_01"], rec["equal_02"]) == expect[k]
        model = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.ReLU(), torch.nn.Linear(4, 4))
        model.load_state_dict({n: torch.tensor(v) for n, v in rec["init"].items()})
        x1 = torch.tensor(rec["x"]).requires_grad_(True)
        y1 = torch.tensor(rec["y"])
        xs = [x1, x1.clone().detach().requires_grad_(True), x1.clone().detach().requires_grad_(True)]
        opt = oracle.StashingOracle("SGD", [model], int(k), lr=1e-1)
        losses = [torch.nn.functional.mse_loss(model(x), y1) for x in xs]
        grads = []
        for loss, x in zip(losses, xs):
            opt.zero_grad()
            opt.load_old_params()
            loss.backward()
            grads.append(x.grad.clone())
            opt.load_new_params()
            opt.step()
        assert torch.equal(grads[0], grads[1]) == rec["equal_01"]
        assert torch.equal(grads[0], grads[2]) == rec["equal_02"]
        for g, ref in zip(grads, rec["x_grads"]):
            assert torch.allclose(g, torch.tensor(ref), rtol=1e-5, atol=1e-7)
        for n, v in model.state_dict().items():
            assert torch.allclose(v, torch.tensor(rec["final"][n]), rtol=1e-5, atol=1e-7)
        assert opt.latest_version == rec["latest_version"]
        assert opt.current_version == rec["current_version"]


@pytest.mark.parametrize("key", sorted(STASH["version_traces_n12"]))
def test_version_traces(key):
    w = int(key.split("_")[0][1:])
    macro = key.endswith("macro1")
    ref = STASH["version_traces_n12"][key]
    assert oracle.version_trace(w, 12, macro) == ref
    # product index logic: VersionRing driven through the same loop
    nv = min(2, w + 1) if macro else w + 1
    interval = nv if macro else 1
    ring = pd_optimizer.VersionRing(nv)
    counter, trace = 0, []
    for kind, i in schedule.stage_program(w, 12):
        if kind == "F":
            trace.append(["F", i, ring.newest()])
        else:
            trace.append(["B", i, ring.oldest() if nv > 1 else ring.newest()])
            if counter % interval == interval - 1:
                ring.advance()
            counter += 1
            trace.append(["S", i, ring.newest()])
    assert trace == ref


def test_version_ring_slots():
    ring = pd_optimizer.VersionRing(3)
    assert ring.versions() == [0, 0, 0]
    seen = []
    for _ in range(7):
        seen.append(ring.advance())
    assert seen == [(0, 1), (1, 2), (2, 0), (0, 1), (1, 2), (2, 0), (0, 1)]
    assert ring.versions() == [5, 6, 7] and ring.oldest() == 5


@pytest.mark.parametrize("name", ["sgd", "adam"])
def test_optimizer_trajectories(name):
    rec = STASH["trajectories"][name]
    m = torch.nn.Linear(8, 8)
    m.load_state_dict({k: torch.tensor(v) for k, v in rec["init"].items()})
    if name == "sgd":
        opt = oracle.StashingOracle("SGD", [m], 2, lr=0.05, momentum=0.9, weight_decay=5e-4)
    else:
        opt = oracle.StashingOracle("Adam", [m], 2, lr=2e-3, weight_decay=1e-4)
    g = torch.Generator().manual_seed(12)
    for s in range(4):
        opt.zero_grad()
        opt.load_old_params()
        for p in m.parameters():
            p.grad = torch.randn(p.shape, generator=g)
        opt.load_new_params()
        opt.step()
        for k, v in m.state_dict().items():
            assert torch.allclose(v, torch.tensor(rec["after_step"][s][k]), rtol=2e-6, atol=1e-7), (name, s, k)


def test_stage_builders_match_golden_weights():
    """Initial weights of the stage builders (seed 0) equal the reference's generated modules:
    the golden run's checksums of never-updated statistics are covered in test_vgg16_pipeline;
    here the product builder and the oracle builder must agree bit for bit."""
    torch.manual_seed(0)
    prod = stages.vgg16("gpus=8").stages()
    torch.manual_seed(0)
    orc = oracle.vgg16_stages("conv4_3")
    for a, b in zip(prod, orc):
        sa, sb = a.state_dict(), b.state_dict()
        assert list(sa) == list(sb)
        assert all(torch.equal(sa[k], sb[k]) for k in sa)


def test_sequence_and_criteria_restatements():
    rng = np.random.RandomState(0)
    x = rng.randn(6, 4, 3).astype(np.float32)
    lengths = [6, 4, 2, 1]
    out = oracle.revert_varlen(x, lengths)
    assert np.array_equal(out[:4, 1], x[:4, 1][::-1]) and np.all(out[4:, 1] == 0)
    m = oracle.set_mask(lengths)
    assert m.shape == (6, 4) and m[:, 2].tolist() == [1, 1, 0, 0, 0, 0]
    logits = rng.randn(12, 50)
    target = rng.randint(0, 50, size=12)
    target[::4] = 0
    t_logits = torch.tensor(logits)
    logp = torch.log_softmax(t_logits, -1)
    mask = torch.tensor(target) != 0
    nll = -logp.gather(1, torch.tensor(target).unsqueeze(1)).squeeze(1)[mask]
    ref = (0.9 * nll + 0.1 * (-logp.mean(-1))[mask]).sum() / 3
    assert abs(oracle.label_smoothing_loss(logits, target, 0, 0.1, 3) - ref.item()) < 1e-9
    ce = torch.nn.functional.cross_entropy(t_logits, torch.tensor(target))
    assert abs(oracle.cross_entropy_loss(logits, target) - ce.item()) < 1e-9


def test_vgg16_pipeline_first_minibatches():
    """Oracle pipeline simulation vs the recorded reference run (2 gloo ranks, 20 minibatches):
    the first minibatches are replayed here; the full 20 are checked on the GPU box."""
    path = os.path.join(GOLD, "vgg16_cfg1_golden.json")
    gold = load("vgg16_cfg1_golden.json")
    cfg = gold["config"]
    n = 3
    torch.manual_seed(cfg["seed"])
    st = oracle.vgg16_stages("conv4_3")
    for s in st:
        oracle.disable_dropout(s)
    model = [(st[0], ["input0"], ["out0"]), (st[1], ["out0"], ["out1"]), (torch.nn.CrossEntropyLoss(), ["out1"], ["loss"])]
    pipe = oracle.PipelineOracle(model, [0, 1, 1], {0: [0], 1: [1]}, None, "SGD",
                                 dict(lr=cfg["lr"], momentum=cfg["momentum"], weight_decay=cfg["weight_decay"]))
    pipe.run({0: stages.SyntheticImages(cfg["batch"], n, seed=cfg["data_seed"])}, n)
    got = pipe.ranks[1]["losses"]
    # with n = 3 the schedule of the first minibatches is the same as in the 20-minibatch run
    for i in range(n):
        assert abs(got[i] - gold["losses"][i]) <= 1e-4 * abs(gold["losses"][i]), (i, got[i], gold["losses"][i])
    for k, key in ((0, "stage0"), (1, "stage1")):
        got_trace = [e for e in pipe.ranks[k]["trace"] if e[0] != "S"]
        assert got_trace[:5] == gold["trace"][key][:5]
