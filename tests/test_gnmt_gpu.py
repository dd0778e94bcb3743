"""Translation path on the GPU: the four GNMT (8+8 layers) stages with native LSTM / embedding / linear /
label-smoothing kernels through StageRuntime and AdamWithWeightStashing, against the golden run of the
reference's own stage modules (tests/golden/gnmt_large_golden.json)."""
import json
import os

import pytest
import torch

# whole-run comparisons: weight gradients without the run-to-run varying split (see conftest.py)
pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("deterministic_weight_gradients")]

from pipedream_b200 import adam, gnmt_blocks, layers, runtime, stages  # noqa: E402
from pipedream_b200 import functional as pf                           # noqa: E402

GOLD = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gnmt_large_golden.json")))


def build(fp16):
    cfg = GOLD["config"]
    torch.manual_seed(cfg["seed"])
    model = stages.gnmt_large().model(gnmt_blocks.LabelSmoothing(0, cfg["smoothing"]))
    for (m, _, _) in model:
        for sub in m.modules():
            if isinstance(sub, torch.nn.Dropout):
                sub.p = 0.0
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


@pytest.mark.parametrize("fp16", [False, True], ids=["fp32", "bf16"])
def test_gnmt_large_three_steps(fp16):
    cfg = GOLD["config"]
    r, opt = build(fp16)
    mods = r.modules()
    assert isinstance(mods[0].layer6, layers.NativeEmbedding)
    assert isinstance(mods[0].layer7, layers.NativeEmuBidirLSTM)
    assert isinstance(mods[0].layer9, layers.NativeLSTM)
    assert isinstance(mods[1].layer24.rnn, layers.NativeLSTM)
    assert isinstance(mods[1].layer24.attn.linear_q, layers.NativeLinear)
    assert isinstance(mods[3].layer13.classifier, layers.NativeLinear)
    assert isinstance(mods[4], layers.NativeLabelSmoothing)
    n = cfg["steps"]
    r.train(n)
    r.set_loader(stages.SyntheticTranslation(cfg["batch"], n, seed=cfg["data_seed"], min_len=cfg["min_len"],
                                             max_len=cfg["max_len"]))
    losses = []
    for _ in range(n):
        r.run_forward()
        losses.append(float(r.tensors[-1]["loss"]))
        opt.zero_grad()
        opt.load_old_params()
        r.run_backward()
        opt.load_new_params()
        opt.step()
    torch.cuda.synchronize()
    assert pf.gemm_poll_error() == 0
    tol = 2e-2 if fp16 else 1e-3
    for i, (a, b) in enumerate(zip(losses, GOLD["losses"])):
        assert abs(a - b) <= tol * abs(b), "step %d: loss %.5f vs reference %.5f" % (i, a, b)
    # updated parameters: checksum per tensor, relative to the tensor's absolute sum
    worst, worst_name = 0.0, None
    for si, m in enumerate(mods[:-1]):
        for k, v in m.state_dict().items():
            ref = GOLD["params"].get("stage%d.%s" % (si, k))
            if ref is None or v is None:
                continue
            if fp16 and k.endswith("normalize_bias"):
                # zero-initialised and updated by Adam, whose step is ~lr * sign(gradient): bf16 rounding of
                # near-zero gradients flips signs, so this 1024-vector is not comparable element-wise
                continue
            t = v.detach().double().flatten()
            e = abs(t.abs().sum().item() - ref["abs_sum"]) / max(ref["abs_sum"], 1e-9)
            if e > worst:
                worst, worst_name = e, "stage%d.%s" % (si, k)
    print("\n[%s] gnmt losses %s vs %s; worst parameter |sum| deviation %.2e" % (
        "bf16" if fp16 else "fp32", [round(x, 4) for x in losses], [round(x, 4) for x in GOLD["losses"]], worst), worst_name)
    assert worst <= (2e-2 if fp16 else 1e-3), worst_name
