"""Translation path on the CPU: the restated GNMT blocks (pipedream_b200/gnmt_blocks.py, plain torch
modules) against the golden run of the reference's own stage modules, and the oracle's explicit LSTM /
attention arithmetic against torch."""
import json
import os

import torch

from oracle import pipedream_oracle as oracle
from pipedream_b200 import gnmt_blocks, stages

GOLD = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gnmt_large_golden.json")))


def test_oracle_lstm_and_attention_arithmetic():
    torch.manual_seed(1)
    lstm = torch.nn.LSTM(12, 8)
    x = torch.randn(5, 3, 12)
    ref, _ = lstm(x)
    got = oracle.lstm_layer(x, lstm.weight_ih_l0, lstm.weight_hh_l0, lstm.bias_ih_l0, lstm.bias_hh_l0)
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-6)
    att = gnmt_blocks.BahdanauAttention(8, 8, 8)
    q, k = torch.randn(2, 4, 8), torch.randn(2, 6, 8)
    ref_s = att.calc_score(q, k)
    got_s = oracle.bahdanau_scores(q, k, att.linear_att, att.normalize_scalar, att.normalize_bias)
    assert torch.allclose(got_s, ref_s, rtol=1e-5, atol=1e-6)


def test_revert_varlen_restatements_agree():
    x = torch.randn(6, 4, 3)
    lengths = torch.tensor([6, 4, 2, 1])
    a = gnmt_blocks._revert_varlen_torch(x, lengths)
    b = torch.from_numpy(oracle.revert_varlen(x.numpy(), lengths.tolist()))
    assert torch.equal(a, b)


def test_synthetic_translation_format():
    (src, src_len), (tgt, tgt_len) = next(iter(stages.SyntheticTranslation(16, 1)))
    assert src.shape == (max(src_len), 16) and tgt.shape == (max(tgt_len), 16)
    assert src_len == sorted(src_len, reverse=True) and min(src_len) >= 20 and max(src_len) <= 50
    assert (src[0] == 2).all() and all(src[L - 1, b] == 3 for b, L in enumerate(src_len))
    assert all((src[L:, b] == 0).all() for b, L in enumerate(src_len))
    body = src[1:min(src_len) - 1]
    assert body.min() >= 4 and body.max() < 32000


def test_gnmt_blocks_reproduce_reference_run():
    """Same seed, data, optimizer as tests/golden/make_golden.py --only gnmt (which runs the reference's
    stage modules): the restated blocks must give the same losses and parameters on the CPU."""
    cfg = GOLD["config"]
    torch.manual_seed(cfg["seed"])
    model = stages.gnmt_large().model(gnmt_blocks.LabelSmoothing(0, cfg["smoothing"]))
    mods = [m for (m, _, _) in model[:-1]]
    for m in mods:
        oracle.disable_dropout(m)
    opt = oracle.StashingOracle("Adam", mods, 1, lr=2e-3, weight_decay=1e-4)
    losses = []
    data = stages.SyntheticTranslation(cfg["batch"], 2, seed=cfg["data_seed"], min_len=cfg["min_len"],
                                       max_len=cfg["max_len"])
    for step, ((src, src_len), (tgt, _)) in enumerate(data):
        t = {"input0": src, "input1": torch.LongTensor(src_len), "input2": tgt[:-1],
             "target": tgt[1:].contiguous().view(-1)}
        for (m, ins, outs) in model:
            if outs == ["loss"]:
                t["loss"] = m(t[ins[0]], t["target"])
            else:
                o = m(*[t[n] for n in ins])
                for n, v in zip(outs, o if isinstance(o, tuple) else (o,)):
                    t[n] = v
        if step == 0:
            for name, ref in GOLD["boundary_tensors_step0"].items():
                got = t[name].detach().double()
                assert abs(got.sum().item() - ref["sum"]) <= 1e-4 * max(1.0, ref["abs_sum"]), name
        opt.zero_grad()
        opt.load_old_params()
        t["loss"].backward()
        opt.load_new_params()
        opt.step()
        losses.append(float(t["loss"]))
    for a, b in zip(losses, GOLD["losses"]):
        assert abs(a - b) <= 1e-4 * abs(b), (losses, GOLD["losses"])
