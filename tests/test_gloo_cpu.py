"""Host logic of StageRuntime + CommunicationHandler over real processes: CPU ranks, gloo transport,
unswapped torch modules (native=False).  Checked against the single-process oracle simulation."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def make_model(seed=0):
    torch.manual_seed(seed)
    s0 = torch.nn.Sequential(torch.nn.Linear(12, 16), torch.nn.Tanh())
    s1 = torch.nn.Sequential(torch.nn.Linear(16, 16), torch.nn.Tanh(), torch.nn.Linear(16, 5))
    return [(s0, ["input0"], ["out0"]), (s1, ["out0"], ["out1"]), (torch.nn.CrossEntropyLoss(), ["out1"], ["loss"])]


class Loader:
    def __init__(self, n, seed, batch=6):
        self.n, self.seed, self.batch = n, seed, batch

    def __iter__(self):
        for i in range(self.n):
            g = torch.Generator().manual_seed(self.seed + i)
            yield torch.randn(self.batch, 12, generator=g), torch.randint(0, 5, (self.batch,), generator=g)


CONFS = {
    "straight2": {"module_to_stage_map": [0, 1, 1], "stage_to_rank_map": {0: [0], 1: [1]}, "stage_to_depth_map": None},
    "hybrid_1_2": {"module_to_stage_map": [0, 1, 1], "stage_to_rank_map": {0: [0], 1: [1, 2]}, "stage_to_depth_map": None},
    "hybrid_2_1": {"module_to_stage_map": [0, 1, 1], "stage_to_rank_map": {0: [0, 1], 1: [2]}, "stage_to_depth_map": None},
}
N0 = 8          # minibatches per stage-0 replica


def worker(rank, world, conf_name, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["PIPEDREAM_MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    from oracle import pipedream_oracle as oracle
    from pipedream_b200 import runtime, schedule
    conf = CONFS[conf_name]
    model = make_model()
    shapes = {"input0": (6, 12), "target": (6,), "out0": (6, 16), "out1": (6, 5)}
    dtypes = {"input0": torch.float32, "target": torch.int64, "out0": torch.float32, "out1": torch.float32}
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import pipeline_util as pu
    pu.register_gloo()
    r = pu.CpuRuntime(model, "gloo", False, 1, shapes, dict(shapes), dtypes, {"input": 0}, {"target"}, conf,
                      "127.0.0.1", rank, 0, 1, 0, runtime.IMAGE_CLASSIFICATION)
    trainable = [m for m in r.modules() if any(True for _ in m.parameters())]
    opt = oracle.StashingOracle("SGD", trainable, r.num_warmup_minibatches + 1, lr=0.1, momentum=0.9)
    sync = getattr(r.modules()[0], "_pd_grad_sync", None)
    orig_step = opt.step

    def step_with_sync():
        if sync is not None:
            for p in opt.params:
                if p.grad is not None:
                    p.grad.mul_(sync(p.grad))
        orig_step()
    opt.step = step_with_sync
    n = r.num_iterations(N0)
    r.train(n)
    r.set_loader(Loader(N0, 100 + 1000 * r.rank_in_stage) if r.stage == 0 else None)
    losses = []
    schedule.train_1f1b(r, opt, n, on_forward=lambda i, rr: losses.append(float(rr.loss)) if rr.is_criterion else None)
    torch.save({"losses": losses, "params": [p.detach().clone() for p in opt.params], "stage": r.stage,
                "rank_in_stage": r.rank_in_stage}, os.path.join(out_dir, "rank%d.pt" % rank))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("conf_name", sorted(CONFS))
def test_runtime_over_gloo_matches_oracle(conf_name, tmp_path):
    from oracle import pipedream_oracle as oracle
    conf = CONFS[conf_name]
    world = sum(len(v) for v in conf["stage_to_rank_map"].values())
    port = 23450 + sorted(CONFS).index(conf_name)
    mp.spawn(worker, args=(world, conf_name, port, str(tmp_path)), nprocs=world, join=True)
    pipe = oracle.PipelineOracle(make_model(), conf["module_to_stage_map"], conf["stage_to_rank_map"], None, "SGD",
                                 dict(lr=0.1, momentum=0.9))
    loaders = {k: Loader(N0, 100 + 1000 * i) for i, k in enumerate(conf["stage_to_rank_map"][0])}
    pipe.run(loaders, N0)
    for rank in range(world):
        got = torch.load(os.path.join(str(tmp_path), "rank%d.pt" % rank))
        ref = pipe.ranks[rank]
        assert len(got["losses"]) == len(ref["losses"])
        for a, b in zip(got["losses"], ref["losses"]):
            assert abs(a - b) <= 1e-6 * max(1.0, abs(b)), (rank, got["losses"], ref["losses"])
        for p, q in zip(got["params"], ref["opt"].params):
            assert torch.allclose(p, q.detach(), rtol=1e-5, atol=1e-7), rank
