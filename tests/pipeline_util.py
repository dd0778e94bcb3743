"""Helpers shared by the GPU tests: build StageRuntime objects the way the driver script does
(runtime/image_classification/main_with_runtime.py:129-229)."""
import torch

import torch.distributed as dist

from pipedream_b200 import runtime, sgd, adam, stages, schedule, communication


# --------------------------------------------------------------------------- #
# test-only variants of the runtime: the product runs native modules on CUDA over peer channels
# --------------------------------------------------------------------------- #
class TorchModuleRuntime(runtime.StageRuntime):
    """StageRuntime whose stage modules stay the user's torch.nn modules (cuDNN / cuBLAS or CPU kernels).
    `device` chooses where they run.  Used as a same-GPU control and for the CPU tests of the host logic."""

    device_override = None

    def _pick_device(self, local_rank):
        if self.device_override is not None:
            return torch.device(self.device_override)
        return torch.device("cuda", local_rank if local_rank is not None else 0)

    def _adopt_module(self, module):
        module = module.to(self.device)
        return module.to(self.compute_dtype) if self.fp16 else module

    def _input_convert(self):
        if self.fp16:
            return lambda x: x.to(self.compute_dtype)      # runtime/runtime.py:397-398
        return None


class CpuRuntime(TorchModuleRuntime):
    device_override = "cpu"


class GlooTransport:
    """CPU ranks over torch.distributed: shape message then payload, like the reference's wire format
    (runtime/communication.py:664-678,704-712), but sends are asynchronous."""

    uses_process_groups = True

    def __init__(self, handler, master_addr, master_port):
        if not dist.is_initialized():
            communication._rendezvous_env(master_addr, master_port)
            dist.init_process_group("gloo", rank=handler.rank, world_size=handler.world_size)
        self.rank = handler.rank
        self.pending = []

    @staticmethod
    def _tag(tag, backward):
        return 2 * tag + (1 if backward else 0)

    def send(self, dst_rank, name, backward, tensor, tag):
        t = tensor.detach().cpu().contiguous()
        shape = torch.tensor(list(t.shape), dtype=torch.int)
        self.pending.append((dist.isend(shape, dst=dst_rank, tag=self._tag(tag, backward)), shape))
        self.pending.append((dist.isend(t, dst=dst_rank, tag=self._tag(tag, backward)), t))
        self.pending = [(w, keep) for (w, keep) in self.pending if not w.is_completed()]

    def recv(self, src_rank, name, backward, shape, dtype, tag):
        got_shape = torch.zeros(len(shape), dtype=torch.int)
        dist.recv(got_shape, src=src_rank, tag=self._tag(tag, backward))
        t = torch.zeros([int(x) for x in got_shape], dtype=dtype)
        dist.recv(t, src=src_rank, tag=self._tag(tag, backward))
        return t

    def wait(self):
        for w, _ in self.pending:
            w.wait()
        self.pending = []


def register_gloo():
    communication.register_transport("gloo", GlooTransport)


def tensor_shapes(model, batch):
    """CPU dry run of every stage on zeros to learn boundary shapes (main_with_runtime.py:142-155)."""
    shapes = {"input0": [batch, 3, 224, 224], "target": [batch]}
    dtypes = {"input0": torch.int64, "target": torch.int64}
    for (stage, inputs, outputs) in model[:-1]:
        ins = [torch.zeros(tuple(shapes[i]), dtype=torch.float32) for i in inputs]
        with torch.no_grad():
            out = stage(*ins)
        out = out if isinstance(out, tuple) else (out,)
        for name, o in zip(outputs, out):
            shapes[name] = list(o.size())
            dtypes[name] = o.dtype
    return {k: tuple(v) for k, v in shapes.items()}, dtypes


def disable_dropout(model):
    for (m, _, _) in model:
        for sub in m.modules():
            if isinstance(sub, torch.nn.Dropout):
                sub.p = 0.0


def make_worker(package, conf, rank, batch, fp16, backend, seed=0, lr=0.01, momentum=0.9, weight_decay=5e-4,
                dropout=False, optimizer="sgd", macrobatch=False, shapes=None, native=True, local_rank=0,
                num_ranks_in_server=1, enable_recompute=False, reference_dtypes=False):
    torch.manual_seed(seed)
    model = package.model(torch.nn.CrossEntropyLoss())
    if not dropout:
        disable_dropout(model)
    if shapes is None:
        shapes = tensor_shapes(model, batch)
    tshapes, dtypes = shapes
    if fp16 and not reference_dtypes:
        # (the reference's driver scripts leave float32 in this table even with --fp16; reference_dtypes=True
        # keeps it that way to check that the runtime substitutes the 16-bit type itself)
        dtypes = {k: (torch.bfloat16 if v == torch.float32 else v) for k, v in dtypes.items()}
    cls = runtime.StageRuntime if native else TorchModuleRuntime
    r = cls(
        model=model, distributed_backend=backend, fp16=fp16, loss_scale=1,
        training_tensor_shapes=dict(tshapes), eval_tensor_shapes=dict(tshapes), training_tensor_dtypes=dtypes,
        inputs_module_destinations={"input": 0}, target_tensor_names={"target"},
        configuration_maps=conf if conf is not None else {"module_to_stage_map": None, "stage_to_rank_map": None,
                                                          "stage_to_depth_map": None},
        master_addr="127.0.0.1", rank=rank, local_rank=local_rank, num_ranks_in_server=num_ranks_in_server,
        verbose_freq=0, model_type=runtime.IMAGE_CLASSIFICATION, enable_recompute=enable_recompute)
    nv = r.num_warmup_minibatches + 1
    if optimizer == "sgd":
        opt = sgd.SGDWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1, num_versions=nv,
                                        lr=lr, momentum=momentum, weight_decay=weight_decay, macrobatch=macrobatch)
    else:
        opt = adam.AdamWithWeightStashing(r.modules(), r.master_parameters, r.model_parameters, 1, num_versions=nv,
                                          lr=lr, weight_decay=weight_decay, macrobatch=macrobatch)
    return r, opt


def local_pipeline(package, conf, batch, fp16, **kw):
    """Every rank of `conf` as a StageRuntime in this process (transport "local")."""
    schedule.reset_local()
    world = sum(len(v) for v in conf["stage_to_rank_map"].values())
    conf = dict(conf)
    conf.setdefault("stage_to_depth_map", None)
    torch.manual_seed(kw.get("seed", 0))
    shapes = tensor_shapes(package.model(torch.nn.CrossEntropyLoss()), batch)
    workers = [make_worker(package, conf, rank, batch, fp16, communication.LOCAL, shapes=shapes, **kw)
               for rank in range(world)]
    return schedule.LocalPipeline(workers)


def param_checksums(r):
    out = {}
    for mi, m in enumerate(r.modules()):
        for k, v in m.state_dict().items():
            t = v.detach().double().flatten().cpu()
            n = t.numel()
            kk = min(8, n)
            idx = torch.tensor([(j * (n - 1)) // max(1, kk - 1) for j in range(kk)], dtype=torch.long)
            out["module%d.%s" % (mi, k)] = {"sum": t.sum().item(), "abs_sum": t.abs().sum().item(),
                                            "sq_sum": (t * t).sum().item(), "samples": t[idx].tolist()}
    return out


def run_cfg1(gold, fp16, native):
    """The golden run's configuration through LocalPipeline; returns (losses, workers).
    native=False keeps the torch.nn modules (cuDNN / cuBLAS) as a same-GPU control."""
    cfg = gold["config"]
    pkg = stages.vgg16("gpus=8")
    pipe = local_pipeline(pkg, pkg.conf, cfg["batch"], fp16, lr=cfg["lr"], momentum=cfg["momentum"],
                          weight_decay=cfg["weight_decay"], seed=cfg["seed"], native=native)
    (r0, o0), (r1, o1) = pipe.workers
    n = cfg["steps"]
    r0.set_loader(stages.SyntheticImages(cfg["batch"], n, seed=cfg["data_seed"]))
    r1.set_loader(None)
    losses = []
    pipe.run([n, n], on_loss=lambda k, i, rr: losses.append(float(rr.loss)))
    return losses, pipe.workers


def checksum_errors(workers, gold):
    """Relative error of the parameter checksums per tensor, split into weights and biases."""
    werr, berr = {}, {}
    for (r, _), key in zip(workers, ("stage0", "stage1")):
        got = param_checksums(r)
        for name, ref in gold["params"][key].items():
            g = got[name]
            scale = max(abs(ref["abs_sum"]), 1e-6)
            e = max(abs(g["sum"] - ref["sum"]), abs(g["abs_sum"] - ref["abs_sum"])) / scale
            (berr if name.endswith("bias") else werr)[key + "." + name] = e
    return werr, berr
