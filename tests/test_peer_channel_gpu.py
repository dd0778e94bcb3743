"""NVLink peer channels: protocol tests on one GPU (producer end opened over the same memory, every
wait already satisfied when it is enqueued), the bounded-wait path, and - where the box has two or
more GPUs - the 2-stage VGG-16 pipeline with one process per GPU."""
import ctypes
import json
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

from pipedream_b200 import _lib  # noqa: E402
from pipedream_b200._lib import call  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _s():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _pair(slot_bytes, slots, timeout_ms):
    cons, prod = ctypes.c_void_p(), ctypes.c_void_p()
    call("pd_chan_create", slot_bytes, slots, timeout_ms, ctypes.byref(cons))
    call("pd_chan_open_local", cons, timeout_ms, ctypes.byref(prod))
    return cons, prod


def test_channel_fifo_and_header():
    n = 1 << 16
    cons, prod = _pair(n * 4, 3, 2000)
    msgs = [torch.full((n,), float(i + 1), device="cuda") for i in range(7)]
    outs = []
    # never more than 3 messages in flight, so no wait has to spin
    for i, m in enumerate(msgs):
        dims = (ctypes.c_int64 * 2)(n // 4, 4)
        call("pd_chan_push", prod, ctypes.c_void_p(m.data_ptr()), n * 4, 2, dims, _s())
        if i >= 2:
            hdr = (ctypes.c_int64 * 8)()
            call("pd_chan_peek_header", cons, hdr, _s())
            assert list(hdr)[:5] == [len(outs) + 1, n * 4, 2, n // 4, 4]
            o = torch.empty(n, device="cuda")
            call("pd_chan_wait", cons, ctypes.c_void_p(o.data_ptr()), n * 4, _s())
            outs.append(o)
    for _ in range(2):
        o = torch.empty(n, device="cuda")
        call("pd_chan_wait", cons, ctypes.c_void_p(o.data_ptr()), n * 4, _s())
        outs.append(o)
    torch.cuda.synchronize()
    for i, o in enumerate(outs):
        assert torch.equal(o, msgs[i])
    assert _lib.load().pd_chan_status(cons, _s()) == 0
    assert _lib.load().pd_chan_status(prod, _s()) == 0
    call("pd_chan_close", prod)
    call("pd_chan_close", cons)


def test_channel_wait_is_bounded():
    """A receive with nothing published gives up after the bound, reports a status, and leaves the
    context usable (this is how a stalled or dead peer shows up).  After that the channel is dead: a second
    queued receive returns at once, `consumed` does not advance, the destination is zero-filled."""
    import time
    cons, prod = _pair(1024, 2, 50)
    o = torch.full((256,), 7.0, device="cuda")
    call("pd_chan_wait", cons, ctypes.c_void_p(o.data_ptr()), 1024, _s())
    rc = _lib.load().pd_chan_status(cons, _s())
    assert rc == -4 and "wait ran out" in _lib.last_error()
    assert _lib.load().pd_chan_poll(cons) == -4                  # host mirror, no synchronisation
    assert (o == 0).all()                                        # not stale slot contents
    t0 = time.time()
    call("pd_chan_wait", cons, ctypes.c_void_p(o.data_ptr()), 1024, _s())
    torch.cuda.synchronize()
    assert time.time() - t0 < 0.04                               # no second 50 ms spin
    assert _lib.load().pd_chan_status(cons, _s()) == -4          # a failed channel stays failed
    # the producer end sees `consumed` still at 0: three pushes into a 2-slot ring must run out as well
    m = torch.ones(256, device="cuda")
    dims = (ctypes.c_int64 * 1)(256)
    for _ in range(3):
        call("pd_chan_push", prod, ctypes.c_void_p(m.data_ptr()), 1024, 1, dims, _s())
    assert _lib.load().pd_chan_status(prod, _s()) == -4
    assert torch.ones(4, device="cuda").sum().item() == 4.0      # the context still works
    # producer side: a full ring that nobody drains
    cons2, prod2 = _pair(1024, 1, 50)
    call("pd_chan_push", prod2, ctypes.c_void_p(m.data_ptr()), 1024, 1, dims, _s())
    call("pd_chan_push", prod2, ctypes.c_void_p(m.data_ptr()), 1024, 1, dims, _s())
    assert _lib.load().pd_chan_status(prod2, _s()) == -4
    with pytest.raises(_lib.PipedreamB200Error):
        call("pd_chan_push", prod2, ctypes.c_void_p(m.data_ptr()), 4096, 1, dims, _s())   # over capacity
    for ch in (prod, cons, prod2, cons2):
        call("pd_chan_close", ch)


def test_channel_size_mismatch_is_an_error():
    """A receive that asks for another byte count than the message carries (the two stages disagree about a
    tensor's shape or element type) fails the channel instead of reinterpreting the payload."""
    cons, prod = _pair(4096, 2, 2000)
    m = torch.ones(512, device="cuda", dtype=torch.bfloat16)          # 1024 bytes
    dims = (ctypes.c_int64 * 1)(512)
    call("pd_chan_push", prod, ctypes.c_void_p(m.data_ptr()), 1024, 1, dims, _s())
    o = torch.full((512,), 3.0, device="cuda")                        # 2048 bytes asked for
    call("pd_chan_wait", cons, ctypes.c_void_p(o.data_ptr()), 2048, _s())
    assert _lib.load().pd_chan_status(cons, _s()) == -1 and "byte count" in _lib.last_error()
    assert (o == 0).all()
    for ch in (prod, cons):
        call("pd_chan_close", ch)


def _pipeline_worker(rank, world, port, out_dir, fp16, reference_dtypes=False):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["PIPEDREAM_MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    torch.backends.cudnn.allow_tf32 = False
    import pipeline_util as pu
    from pipedream_b200 import schedule, stages
    gold = json.load(open(os.path.join(ROOT, "tests", "golden", "vgg16_cfg1_golden.json")))
    cfg = gold["config"]
    pkg = stages.vgg16("gpus=8")
    conf = dict(pkg.conf)
    conf["stage_to_depth_map"] = None
    r, opt = pu.make_worker(pkg, conf, rank, cfg["batch"], fp16, "p2p", lr=cfg["lr"], momentum=cfg["momentum"],
                            weight_decay=cfg["weight_decay"], seed=cfg["seed"], local_rank=rank,
                            reference_dtypes=reference_dtypes)
    n = cfg["steps"]
    r.train(n)
    r.set_loader(stages.SyntheticImages(cfg["batch"], n, seed=cfg["data_seed"]) if r.stage == 0 else None)
    losses = []
    schedule.train_1f1b(r, opt, n, on_forward=lambda i, rr: losses.append(float(rr.loss)) if rr.is_criterion else None)
    torch.cuda.synchronize()
    werr, berr = pu.checksum_errors([(r, opt)], {"params": {"stage0": gold["params"]["stage%d" % r.stage]}})
    json.dump({"losses": losses, "werr": max(werr.values()), "berr": max(berr.values())},
              open(os.path.join(out_dir, "rank%d.json" % rank), "w"))
    import torch.distributed as dist
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("fp16", [False, True], ids=["fp32", "bf16"])
def test_two_stage_pipeline_over_peer_channels(fp16, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_pipeline_worker, args=(2, 24500 + int(fp16), str(tmp_path), fp16), nprocs=2, join=True)
    gold = json.load(open(os.path.join(ROOT, "tests", "golden", "vgg16_cfg1_golden.json")))
    got = json.load(open(os.path.join(str(tmp_path), "rank1.json")))
    rel = [abs(a - b) / abs(b) for a, b in zip(got["losses"], gold["losses"])]
    tol = 2e-2 if fp16 else 1e-3
    assert len(rel) == 20 and max(rel[:5]) <= tol, rel
    # same bound as the single-process pipeline test (the fp32 noise floor of this network, see there)
    assert max(rel) <= max(tol, 1.2e-2), rel
    for rank in (0, 1):
        g = json.load(open(os.path.join(str(tmp_path), "rank%d.json" % rank)))
        assert g["werr"] <= max(tol, 5e-3), g


def test_sixteen_bit_pipeline_with_the_drivers_float32_dtype_table(tmp_path):
    """The reference's driver scripts record float32 for every boundary tensor even when they run with --fp16
    (main_with_runtime.py:139-155).  The stages then push bf16; the receiver must allocate and copy bf16 too (a
    float32 receive of twice the bytes would reinterpret the payload - and now fails the channel on the byte count)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_pipeline_worker, args=(2, 24510, str(tmp_path), True, True), nprocs=2, join=True)
    gold = json.load(open(os.path.join(ROOT, "tests", "golden", "vgg16_cfg1_golden.json")))
    got = json.load(open(os.path.join(str(tmp_path), "rank1.json")))
    rel = [abs(a - b) / abs(b) for a, b in zip(got["losses"], gold["losses"])]
    assert len(rel) == 20 and max(rel) <= 2e-2, rel


def _gnmt_worker(rank, world, port, out_dir):
    """Stages 0-1 on GPU 0, stages 2-3 and the criterion on GPU 1, no input pipelining (one version),
    so the arithmetic is that of the single-process golden run."""
    sys.path.insert(0, ROOT)
    os.environ["PIPEDREAM_MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    from pipedream_b200 import adam, gnmt_blocks, runtime, schedule, stages
    gold = json.load(open(os.path.join(ROOT, "tests", "golden", "gnmt_large_golden.json")))
    cfg = gold["config"]
    torch.manual_seed(cfg["seed"])
    model = stages.gnmt_large().model(gnmt_blocks.LabelSmoothing(0, cfg["smoothing"]))
    for (m, _, _) in model:
        for sub in m.modules():
            if isinstance(sub, torch.nn.Dropout):
                sub.p = 0.0
    B, Tm, H, V = cfg["batch"], cfg["max_len"], 1024, 32320
    shapes = {"input0": (Tm, B), "input1": (B,), "input2": (Tm, B), "target": (Tm * B,), "target_length": (B,),
              "out0": (Tm, B, H), "out1": (Tm, B, H), "out12": (Tm, B, H), "out13": (Tm, B, H), "out14": (Tm, B, H),
              "out15": (Tm, B, 2 * H), "out12again": (Tm, B, H), "out18": (Tm, B, V)}
    dtypes = {k: torch.float32 for k in shapes}
    dtypes.update({"input0": torch.int64, "input1": torch.int64, "input2": torch.int64, "target": torch.int64,
                   "target_length": torch.int64})
    conf = {"module_to_stage_map": [0, 0, 1, 1, 1], "stage_to_rank_map": {0: [0], 1: [1]}, "stage_to_depth_map": None}
    r = runtime.StageRuntime(
        model=model, distributed_backend="p2p", fp16=False, loss_scale=1, training_tensor_shapes=shapes,
        eval_tensor_shapes=dict(shapes), training_tensor_dtypes=dtypes,
        inputs_module_destinations={"input0": 0, "input1": 1, "input2": 1},
        target_tensor_names={"target", "target_length"}, configuration_maps=conf, master_addr="127.0.0.1",
        rank=rank, local_rank=rank, num_ranks_in_server=1, verbose_freq=0, model_type=runtime.TRANSLATION)
    opt = adam.AdamWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1, num_versions=1,
                                      lr=2e-3, weight_decay=1e-4)
    n = cfg["steps"]
    r.train(n)
    r.set_loader(stages.SyntheticTranslation(B, n, seed=cfg["data_seed"], min_len=cfg["min_len"], max_len=Tm)
                 if r.stage == 0 else None)
    losses = []
    schedule.train_1f1b(r, opt, n, no_input_pipelining=True,
                        on_forward=lambda i, rr: losses.append(float(rr.tensors[-1]["loss"])) if rr.is_criterion else None)
    torch.cuda.synchronize()
    json.dump({"losses": losses}, open(os.path.join(out_dir, "rank%d.json" % rank), "w"))
    import torch.distributed as dist
    dist.barrier()
    dist.destroy_process_group()


def test_gnmt_two_gpus_variable_length_batches(tmp_path):
    """Translation stages over the peer channels: boundary tensors change shape every minibatch, model
    inputs (lengths, decoder tokens) and targets are forwarded to the later stage."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_gnmt_worker, args=(2, 24510, str(tmp_path)), nprocs=2, join=True)
    gold = json.load(open(os.path.join(ROOT, "tests", "golden", "gnmt_large_golden.json")))
    got = json.load(open(os.path.join(str(tmp_path), "rank1.json")))
    assert len(got["losses"]) == len(gold["losses"])
    for a, b in zip(got["losses"], gold["losses"]):
        assert abs(a - b) <= 1e-3 * abs(b), (got["losses"], gold["losses"])
