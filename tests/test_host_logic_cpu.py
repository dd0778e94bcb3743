"""Host-side logic that needs no GPU: the drop-in modules keep the reference's signatures, boundary routing and
tensor tags equal the reference's for every benchmark stage/rank map, the 16-bit element-type rule, which
boundary tensors carry gradients, and the per-stage minibatch arithmetic of replicated pipelines."""
import inspect
import json
import os

import pytest
import torch

from pipedream_b200 import communication, runtime
from pipedream_b200.dropin import adam as d_adam, optimizer as d_optimizer, runtime as d_runtime, sgd as d_sgd

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SIG = json.load(open(os.path.join(GOLD, "signatures_golden.json")))
ROUTING = json.load(open(os.path.join(GOLD, "routing_golden.json")))


def _sig(fn):
    out = []
    for name, p in inspect.signature(fn).parameters.items():
        if name == "self":
            continue
        out.append([name, None if p.default is inspect.Parameter.empty else repr(p.default)])
    return out


def test_dropin_modules_keep_the_reference_signatures():
    """`import runtime, sgd, adam` in main_with_runtime.py (runtime/image_classification/main_with_runtime.py:25-27)
    must find the same classes, constructor arguments (names, order, defaults) and methods."""
    classes = {"runtime.StageRuntime": d_runtime.StageRuntime, "sgd.SGDWithWeightStashing": d_sgd.SGDWithWeightStashing,
               "adam.AdamWithWeightStashing": d_adam.AdamWithWeightStashing,
               "optimizer.OptimizerWithWeightStashing": d_optimizer.OptimizerWithWeightStashing}
    for key, cls in classes.items():
        for method, want in SIG[key].items():
            assert hasattr(cls, method), "%s.%s is missing" % (key, method)
            got = _sig(getattr(cls, method))
            # an implementation may append arguments of its own after the reference's, never change those
            assert got[:len(want)] == want, "%s.%s: %s vs reference %s" % (key, method, got, want)
    for name, value in SIG["runtime.constants"].items():
        assert getattr(d_runtime, name) == value


@pytest.mark.parametrize("cfg", sorted(ROUTING))
def test_boundary_routing_and_tags_match_the_reference(cfg):
    g = ROUTING[cfg]
    m2s = g["module_to_stage_map"]
    s2r = {int(k): v for k, v in g["stage_to_rank_map"].items()}
    n_model = len(m2s)
    names = ["input0"] + ["out%d" % i for i in range(n_model - 1)]
    model = [(None, [names[i]], [names[i + 1]]) for i in range(n_model - 1)] + [(None, [names[-1]], ["loss"])]
    for rec in g["ranks"]:
        recv, send, fwd = runtime.boundary_routing(model, m2s, s2r, rec["stage"], {"input": 0})
        tags = runtime.assign_tensor_tags(model, {"target"})
        # the handler adds the targets to the rank maps it shares with the runtime (communication.py:165-188)
        if rec["ranks_in_previous_stage"]:
            recv["target"] = rec["ranks_in_previous_stage"]
        if rec["ranks_in_next_stage"]:
            send["target"] = rec["ranks_in_next_stage"]
        assert recv == rec["receive_ranks"], (cfg, rec["rank"])
        assert send == rec["send_ranks"], (cfg, rec["rank"])
        assert tags == rec["tensor_tags"], (cfg, rec["rank"])
        assert fwd == []


def test_forwarded_model_inputs_travel_hop_by_hop():
    """GNMT: the source lengths and the decoder inputs are model inputs that stage 1 consumes; the stages before it
    pass them on (runtime/runtime.py:208-222)."""
    model = [(None, ["input0", "input1"], ["out0"]), (None, ["out0", "input1", "input2"], ["out1"]),
             (None, ["out1"], ["out2"]), (None, ["out2"], ["loss"])]
    m2s, s2r = [0, 1, 2, 2], {0: [0], 1: [1], 2: [2]}
    dest = {"input0": 0, "input1": 1, "input2": 1}
    r0, s0, f0 = runtime.boundary_routing(model, m2s, s2r, 0, dest)
    r1, s1, _ = runtime.boundary_routing(model, m2s, s2r, 1, dest)
    r2, s2, _ = runtime.boundary_routing(model, m2s, s2r, 2, dest)
    assert s0 == {"out0": [1], "input1": [1], "input2": [1]} and r0 == {}
    assert r1 == {"out0": [0], "input1": [0], "input2": [0]} and s1 == {"out1": [2]}
    assert r2 == {"out1": [1]} and s2 == {}
    assert sorted(f0) == ["input1", "input2"]


def test_sixteen_bit_runs_substitute_the_element_type():
    """The driver scripts record float32 for every boundary tensor even with --fp16 (main_with_runtime.py:139-155);
    the handler must then move the 16-bit type (the reference does the same, runtime/communication.py:273)."""
    dtypes = {"out0": torch.float32, "input1": torch.int64, "target": torch.int64}
    for fp16, want in ((True, torch.bfloat16), (False, torch.float32)):
        h = communication.CommunicationHandler("127.0.0.1", 12345, 0, 0, 1, 2, fp16, communication.LOCAL)
        h.initialize({}, {"out0": [1]}, {"out0": 1, "target": 2, "ack": 3}, {"target"}, dtypes, 0, 1, [], [1])
        assert h._dtype("out0") == want
        assert h._dtype("input1") == torch.int64 and h._dtype("target") == torch.int64 and h._dtype("ack") == torch.int64
        assert h._dtype("not recorded") == torch.int64


def test_unknown_backend_is_refused():
    with pytest.raises(ValueError) as e:
        communication.CommunicationHandler("127.0.0.1", 12345, 0, 0, 1, 2, False, "gloo")
    assert "peer channels" in str(e.value)


def test_replicated_gnmt_minibatch_counts_divide():
    """Four stages x two replicas: every rank's message counts per peer must be whole numbers
    (runtime/communication.py:222-248); an odd count per replica is rejected up front."""
    s2r = {0: [0, 1], 1: [2, 3], 2: [4, 5], 3: [6, 7]}
    conf = {"module_to_stage_map": [0, 1, 2, 3, 3], "stage_to_rank_map": s2r, "stage_to_depth_map": None}
    for rank in range(8):
        a = runtime.stage_assignment(5, conf, rank)
        assert a["num_warmup_minibatches"] == (7 - 2 * a["stage"]) // 2
        h = communication.CommunicationHandler("127.0.0.1", 12345, rank, 0, 1, 8, True, communication.LOCAL)
        h.initialize({}, {}, {"ack": 1}, set(), {}, a["rank_in_stage"], 2, a["ranks_in_previous_stage"], a["ranks_in_next_stage"])
        assert h.num_iterations_for_helper_threads(46) == (23 if a["ranks_in_next_stage"] else 0,
                                                           23 if a["ranks_in_previous_stage"] else 0)
        if a["ranks_in_next_stage"] or a["ranks_in_previous_stage"]:
            with pytest.raises(AssertionError):
                h.num_iterations_for_helper_threads(45)
