"""Stage runtime behind the interface of the reference's runtime/runtime.py:44-680.

`StageRuntime` keeps the constructor signature, methods and attributes that
main_with_runtime.py uses (`train`, `eval`, `set_loader`, `run_forward`,
`run_backward`, `run_ack`, `wait`, `num_iterations`,
`get_adjusted_learning_rate`, `state_dict`, `load_state_dict`, `modules`,
`parameters`, `zero_grad`, `stage`, `num_stages`, `num_ranks`,
`num_warmup_minibatches`, `rank_in_stage`, `num_ranks_in_first_stage`,
`master_parameters`, `model_parameters`, `output`, `target`, `loss`).

How it works is its own design:

* `StagePlan` is derived once from the `(module, inputs, outputs)` list: the ordered
  steps of this stage, which tensors enter it, which leave it and which of those
  carry a gradient.  A minibatch is then a short loop over the plan - nothing is
  re-derived per minibatch.
* Tensors that arrive from the previous stage are autograd leaves; after the
  backward pass their `.grad` is what travels back.  Boundary tensors that are not
  floating point (sequence lengths, decoder inputs forwarded hop by hop) get no
  gradient message at all - the reference sends the tensor itself back as a
  placeholder (runtime/runtime.py:611-618).
* Stage 0 reads its loader one minibatch ahead and uploads it on a copy stream, so
  the host-to-device transfer overlaps the previous minibatch's kernels.
* `enable_recompute` is honoured (the reference only stores the flag,
  runtime/runtime.py:72-78): the forward pass runs without an autograd graph and
  keeps only the stage inputs; the backward pass first re-runs the forward on the
  stashed weight version the optimizer has loaded, then back-propagates.
* The stage's leaf modules are swapped for CUDA-native ones (layers.nativize),
  boundary tensors move over NVLink peer channels, and a replicated stage averages
  its flat gradient arena over NCCL instead of DistributedDataParallel.
"""
import collections
import itertools
import os
import weakref

import torch
import torch.distributed as dist

from . import communication
from . import layers
from . import runtime_utilities

IMAGE_CLASSIFICATION = "image_classification"
TRANSLATION = "translation"
SPEECH_TO_TEXT = "speech_to_text"

_MODEL_INPUT_NAMES = ("input0", "input1", "input2", "input")


# --------------------------------------------------------------------------- #
# stage / rank arithmetic
# --------------------------------------------------------------------------- #
def stage_assignment(num_modules, configuration_maps, rank):
    """Which modules, stage, replica index and warm-up depth `rank` gets - the arithmetic of
    runtime/runtime.py:129-175 as a pure function (the CPU tests compare it with values recorded
    from the reference).  Returns a dict."""
    m2s = configuration_maps['module_to_stage_map']
    s2r = configuration_maps['stage_to_rank_map']
    depth = configuration_maps.get('stage_to_depth_map')
    if len(m2s) != num_modules:
        raise AssertionError("module_to_stage_map has %d entries for %d modules" % (len(m2s), num_modules))
    stage_of_rank = {r: s for s, ranks in s2r.items() for r in ranks}
    if rank not in stage_of_rank:
        raise AssertionError("rank %r is not in stage_to_rank_map" % (rank,))
    stage = stage_of_rank[rank]
    num_stages = len(set(m2s))
    replicas = s2r[stage]
    out = {
        "num_ranks": len(stage_of_rank),
        "num_stages": num_stages,
        "stage": stage,
        "rank_in_stage": replicas.index(rank),
        "num_ranks_in_stage": len(replicas),
        "num_ranks_in_first_stage": len(s2r[0]),
        "ranks_in_previous_stage": list(s2r[stage - 1]) if stage > 0 else [],
        "ranks_in_next_stage": list(s2r[stage + 1]) if stage + 1 < num_stages else [],
        "modules": [i for i, s in enumerate(m2s) if s == stage],
        "is_criterion": stage == num_stages - 1,
    }
    if depth is not None:
        out["num_warmup_minibatches"] = depth[str(stage)]       # keys are strings (runtime/runtime.py:167-168)
    else:
        # ranks in later stages, shared between this stage's replicas
        later = out["num_ranks"] - 1 - sum(len(s2r[s]) for s in range(stage))
        out["num_warmup_minibatches"] = later // len(replicas)
    return out


def boundary_routing(model, module_to_stage_map, stage_to_rank_map, stage, inputs_module_destinations):
    """(receive_ranks, send_ranks) of `stage`: for every tensor that crosses a stage boundary the ranks that
    produce / consume it (runtime/runtime.py:192-222).  Model inputs needed by a later stage travel hop by
    hop through the stages in between.  Also returns the model inputs that need a tag of their own."""
    receive, send = {}, {}
    consumers = collections.defaultdict(list)            # tensor -> stages that read it, in module order
    for j, (_, ins, _) in enumerate(model):
        for name in ins:
            consumers[name].append((j, module_to_stage_map[j]))
    for i, (_, _, outs) in enumerate(model):
        src = module_to_stage_map[i]
        for name in outs:
            for j, dst in consumers.get(name, ()):
                if j <= i or dst == src:
                    continue
                if dst == stage:
                    receive[name] = stage_to_rank_map[src]
                if src == stage:
                    send[name] = stage_to_rank_map[dst]
    forwarded = []
    num_stages = len(stage_to_rank_map)
    for name, module in inputs_module_destinations.items():
        dst = module_to_stage_map[module]
        if dst > stage:
            send[name] = stage_to_rank_map[stage + 1] if stage + 1 < num_stages else []
        if 0 < stage <= dst:
            receive[name] = stage_to_rank_map[stage - 1]
        if dst > 0:
            forwarded.append(name)
    return receive, send, forwarded


def assign_tensor_tags(model, target_tensor_names):
    """Tags 1, 2, ... in first-appearance order, then the targets in sorted order, then "ack"
    (runtime/runtime.py:93-110)."""
    tags = {}
    for (_, ins, outs) in model:
        for name in itertools.chain(ins, outs):
            tags.setdefault(name, len(tags) + 1)
    for name in sorted(target_tensor_names):
        tags[name] = len(tags) + 1
    tags["ack"] = len(tags) + 1
    return tags


class StagePlan:
    """What one stage does per minibatch, derived once from its `(module, inputs, outputs)` entries."""

    def __init__(self, entries, is_criterion):
        self.modules = [m for (m, _, _) in entries]
        self.steps = []
        produced, consumed = [], []
        for k, (_, ins, outs) in enumerate(entries):
            self.steps.append((k, tuple(ins), tuple(outs), is_criterion and k == len(entries) - 1))
            consumed.extend(ins)
            produced.extend(outs)
        pset, cset = set(produced), set(consumed)
        # tensors the stage reads but does not make / makes but does not read itself
        self.inputs = [n for n in dict.fromkeys(consumed) if n not in pset]
        self.outputs = [n for n in dict.fromkeys(produced) if n not in cset]
        self.all_input_names = [list(ins) for (_, ins, _) in entries]
        self.all_output_names = [list(outs) for (_, _, outs) in entries]
        self.last_inputs = tuple(entries[-1][1])
        self.last_outputs = tuple(entries[-1][2])

    def run(self, tensors):
        """Runs the steps in order over the name -> tensor dict (filled in place)."""
        mods = self.modules
        for k, ins, outs, criterion in self.steps:
            if criterion:
                total = None
                for name in ins:
                    term = mods[k](tensors[name], tensors["target"])
                    total = term if total is None else total + term
                tensors[outs[0]] = total
                continue
            result = mods[k](*[tensors[name] for name in ins])
            if not isinstance(result, tuple):
                result = (result,)
            for name, value in zip(outs, result):
                tensors[name] = value


class ModulesWithDependencies:
    """Accessor object with the reference's method names (runtime/runtime.py:17-42) over a StagePlan."""

    def __init__(self, plan):
        self._plan = plan

    def modules(self):
        return self._plan.modules

    def all_input_names(self):
        return self._plan.all_input_names

    def all_output_names(self):
        return self._plan.all_output_names

    def is_input_tensor(self, tensor_name):
        return any(tensor_name in names for names in self._plan.all_input_names)


# --------------------------------------------------------------------------- #
# input feeder (stage 0)
# --------------------------------------------------------------------------- #
class InputFeeder:
    """Turns loader items into the stage's input dict, one minibatch ahead of its use.

    Image batches are `(input, target)`; translation batches are `((src, src_len), (tgt, tgt_len))`
    (runtime/runtime.py:380-400).  The upload of minibatch i+1 is issued on a copy stream while
    minibatch i computes; `next()` makes the compute stream wait for the upload it hands out.
    """

    def __init__(self, loader, model_type, device, target_length_dtype, convert=None):
        self.it = iter(loader)
        self.model_type = model_type
        self.device = device
        self.target_length_dtype = target_length_dtype
        self.convert = convert
        self.stream = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        self.ahead = None
        self._fetch()

    def _names(self, item):
        if self.model_type == TRANSLATION:
            (src, src_length), (tgt, tgt_length) = item
            tgt_length = torch.as_tensor(tgt_length, dtype=torch.int64)
            return {
                "input0": src,
                "input1": torch.as_tensor(src_length, dtype=torch.int64),
                "input2": tgt[:-1],
                "target": tgt[1:].contiguous().view(-1),
                "target_length": torch.tensor([int((tgt_length - 1).sum())], dtype=self.target_length_dtype),
            }
        if self.model_type == IMAGE_CLASSIFICATION:
            inp, target = item
            if self.convert is not None:
                inp = self.convert(inp)
            return {"input0": inp, "target": target}
        raise NotImplementedError("model_type %r is not supported" % (self.model_type,))

    def _fetch(self):
        try:
            item = next(self.it)
        except StopIteration:
            self.ahead = None
            return
        host = self._names(item)
        if self.stream is None:
            self.ahead = ({k: v.to(self.device) for k, v in host.items()}, None)
            return
        with torch.cuda.stream(self.stream):
            dev = {k: v.to(self.device, non_blocking=True) for k, v in host.items()}
            done = torch.cuda.Event()
            done.record(self.stream)
        self.ahead = (dev, done)

    def next(self):
        if self.ahead is None:
            raise StopIteration
        dev, done = self.ahead
        if done is not None:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_event(done)
            for t in dev.values():
                t.record_stream(cur)
        self._fetch()
        return dev


# --------------------------------------------------------------------------- #
# the runtime
# --------------------------------------------------------------------------- #
class StageRuntime:
    def __init__(self, model, distributed_backend, fp16, loss_scale,
                 training_tensor_shapes, eval_tensor_shapes,
                 training_tensor_dtypes, inputs_module_destinations,
                 target_tensor_names, configuration_maps, master_addr,
                 rank, local_rank, num_ranks_in_server, verbose_freq,
                 model_type, enable_recompute=False):
        """Arguments are the reference's (runtime/runtime.py:45-50).  `fp16=True` selects 16-bit compute,
        which on this hardware is bf16 with fp32 master weights inside the optimizer.  The stage runs on
        CUDA device `local_rank` with the native kernels; without the CUDA library or an sm_100 device the
        constructor raises."""
        self.tensors = []
        self.gradients = {}
        self.distributed_backend = distributed_backend
        self.fp16 = fp16
        self.loss_scale = loss_scale
        self.training_tensor_shapes = training_tensor_shapes
        self.eval_tensor_shapes = eval_tensor_shapes
        self.training_tensor_dtypes = training_tensor_dtypes
        self.model_type = model_type
        self.target_tensor_names = target_tensor_names
        self.compute_dtype = torch.bfloat16 if fp16 else torch.float32
        self.device = self._pick_device(local_rank)
        self.loader_iter = None
        self._feeder = None
        self._optimizer_ref = None

        self.initialize(model, inputs_module_destinations, configuration_maps,
                        master_addr, rank, local_rank, num_ranks_in_server)

        self.verbose_freq = verbose_freq
        self.forward_only = False
        self.forward_stats = runtime_utilities.RuntimeStats(forward=True)
        self.backward_stats = runtime_utilities.RuntimeStats(forward=False)
        # The last rank of a server never recomputes (runtime/runtime.py:76-78): its backward pass follows
        # its forward pass at once, so nothing would be saved.
        self.enable_recompute = bool(enable_recompute) and rank != num_ranks_in_server - 1

    # ------------------------------------------------------------------ hooks a host-logic test may override
    def _pick_device(self, local_rank):
        if not torch.cuda.is_available():
            raise RuntimeError("pipedream_b200.StageRuntime needs a CUDA device (there is no CPU path)")
        from . import _lib
        _lib.load()               # fail now, loudly, if the CUDA library was not built
        dev = torch.device("cuda", local_rank if local_rank is not None else 0)
        torch.cuda.set_device(dev)
        _lib.call("pd_device_ok")
        return dev

    def _adopt_module(self, module):
        """Moves a user module to the device / compute dtype and swaps its leaves for native ones."""
        module = module.to(self.device)
        if self.fp16:
            module = module.to(self.compute_dtype)
        return layers.nativize(module)

    def _input_convert(self):
        return None      # native stages convert the image batch inside their first kernel

    # ------------------------------------------------------------------ set-up
    def initialize(self, model, inputs_module_destinations, configuration_maps,
                   master_addr, rank, local_rank, num_ranks_in_server):
        self.rank = rank
        self.local_rank = local_rank
        self.forward_minibatch_id = 0
        self.backward_minibatch_id = 0
        self.criterion_input_name = str(model[-1][1][0])
        self.tensor_tags = assign_tensor_tags(model, self.target_tensor_names)
        self.send_ranks = {}
        self.receive_ranks = {}

        module_to_stage_map = configuration_maps['module_to_stage_map']
        stage_to_rank_map = configuration_maps['stage_to_rank_map']
        if module_to_stage_map is None:
            # one process runs every module; nothing is communicated (runtime/runtime.py:113-127)
            if self.rank is not None:
                raise AssertionError("rank must be None without a module_to_stage_map")
            a = {"num_ranks": 1, "num_stages": 1, "stage": None, "rank_in_stage": 0, "num_ranks_in_stage": 1,
                 "num_ranks_in_first_stage": 1, "ranks_in_previous_stage": [], "ranks_in_next_stage": [],
                 "modules": list(range(len(model))), "is_criterion": True, "num_warmup_minibatches": 0}
        else:
            if self.rank is None:
                raise AssertionError("a module_to_stage_map needs a rank")
            a = stage_assignment(len(model), configuration_maps, self.rank)
        self.num_ranks = a["num_ranks"]
        self.num_stages = a["num_stages"]
        self.stage = a["stage"]
        self.rank_in_stage = a["rank_in_stage"]
        self.num_ranks_in_stage = a["num_ranks_in_stage"]
        self.num_ranks_in_first_stage = a["num_ranks_in_first_stage"]
        self.ranks_in_previous_stage = a["ranks_in_previous_stage"]
        self.num_ranks_in_previous_stage = len(self.ranks_in_previous_stage)
        self.ranks_in_next_stage = a["ranks_in_next_stage"]
        self.num_ranks_in_next_stage = len(self.ranks_in_next_stage)
        self.is_criterion = a["is_criterion"]
        self.num_warmup_minibatches = a["num_warmup_minibatches"]

        self.comm_handler = None
        if module_to_stage_map is not None:
            # fixed port of the reference (runtime/runtime.py:181); overridable for concurrent jobs
            master_port = int(os.environ.get("PIPEDREAM_MASTER_PORT", "12345"))
            self.comm_handler = communication.CommunicationHandler(
                master_addr=master_addr, master_port=master_port, rank=self.rank,
                local_rank=self.local_rank, num_ranks_in_server=num_ranks_in_server,
                world_size=self.num_ranks, fp16=self.fp16, backend=self.distributed_backend)
            self.receive_ranks, self.send_ranks, forwarded = boundary_routing(
                model, module_to_stage_map, stage_to_rank_map, self.stage, inputs_module_destinations)
            for name in forwarded:
                self.tensor_tags.setdefault(name, len(self.tensor_tags) + 1)

        entries = [(self._adopt_module(model[i][0]), model[i][1], model[i][2]) for i in a["modules"]]
        self.plan = StagePlan(entries, self.is_criterion)
        self.modules_with_dependencies = ModulesWithDependencies(self.plan)

        # Replicated stages: one process group per stage, created in the same order on every rank.
        self.stage_group = None
        if stage_to_rank_map is not None and self.comm_handler.uses_process_groups():
            groups = []
            for stage in range(self.num_stages):
                ranks = stage_to_rank_map[stage]
                groups.append(dist.new_group(ranks=ranks) if len(ranks) > 1 else None)
            self.stage_group = groups[self.stage]
        if self.num_ranks_in_stage > 1:
            num_parameters = sum(p.numel() for p in self.parameters())
            print("Replicating stage: ranks=%d, module_size=%.3f" % (
                self.num_ranks_in_stage, 4. * num_parameters))
            sync = GradientAverager(self.stage_group, self.num_ranks_in_stage)
            for m in self.plan.modules:
                m._pd_grad_sync = sync
            self._warn_replicated_batchnorm()

        # 16-bit master weights live inside the optimizer's arena, so the two lists of the
        # reference (apex prep_param_lists, runtime/runtime.py:268-276) collapse into one.
        self.master_parameters = list(self.parameters())
        self.model_parameters = None
        for m in self.plan.modules:
            m._pd_runtime = weakref.ref(self)

        if self.comm_handler is not None:
            self.comm_handler.variable_shapes = (self.model_type == TRANSLATION)
            self.comm_handler.initialize(
                self.receive_ranks, self.send_ranks, self.tensor_tags,
                self.target_tensor_names, self.training_tensor_dtypes,
                self.rank_in_stage, self.num_ranks_in_stage,
                self.ranks_in_previous_stage, self.ranks_in_next_stage)

    def _warn_replicated_batchnorm(self):
        """DistributedDataParallel broadcasts rank 0's BatchNorm running statistics at every forward
        (runtime/runtime.py:258-262); here each replica keeps its own until `state_dict()`, which
        takes replica 0's (see `sync_replica_buffers`)."""
        self._replicated_buffers = any(True for m in self.plan.modules for _ in m.buffers())

    def sync_replica_buffers(self):
        """Broadcast replica 0's module buffers (BatchNorm running statistics) to the other replicas
        of this stage.  Called before evaluation and before a checkpoint is taken."""
        if self.stage_group is None or not getattr(self, "_replicated_buffers", False):
            return
        src = dist.get_global_rank(self.stage_group, 0)
        for m in self.plan.modules:
            for b in m.buffers():
                dist.broadcast(b, src=src, group=self.stage_group)

    # ------------------------------------------------------------------ accessors
    @property
    def target(self):
        return self.tensors[-1]["target"]

    def modules(self):
        return self.plan.modules

    def parameters(self):
        return itertools.chain(*[m.parameters() for m in self.plan.modules])

    def state_dict(self):
        """{"module<i>": module.state_dict()} as runtime/runtime.py:306-309 writes it."""
        self.sync_replica_buffers()
        out = collections.OrderedDict()
        for i, module in enumerate(self.plan.modules):
            out["module%d" % i] = module.state_dict()
        return out

    def load_state_dict(self, state_dict):
        """Loads every module (runtime/runtime.py:311-312).  When an optimizer has already taken the stage's
        parameters into its version ring, the ring and the fp32 master copy are re-seeded from the loaded
        values (every stashed version becomes the loaded one, as at construction)."""
        for i, module in enumerate(self.plan.modules):
            module.load_state_dict(state_dict["module%d" % i])
        opt = self._optimizer_ref() if self._optimizer_ref is not None else None
        if opt is not None:
            opt.resync_from_modules()

    def attach_optimizer(self, optimizer):
        self._optimizer_ref = weakref.ref(optimizer)

    def cuda(self):
        for i, m in enumerate(self.plan.modules):
            self.plan.modules[i] = m.to(self.device)

    def zero_grad(self):
        for p in self.parameters():
            p._pd_acc = False
            if p.grad is not None and p.grad is not getattr(p, "_pd_grad", None):
                p.grad = None

    # ------------------------------------------------------------------ epoch control
    def _carries_gradient(self, name):
        """A boundary tensor has a gradient message iff it is floating point (decided from the dtype table
        both neighbours share, so producer and consumer always agree)."""
        if name in self.target_tensor_names or name == "ack":
            return False
        dtype = self.training_tensor_dtypes.get(name)
        return dtype is not None and dtype.is_floating_point

    def _start(self, num_iterations, shapes, forward_only):
        self.tensors = []
        self.gradients = {}
        self.tensor_shapes = shapes
        self.forward_only = forward_only
        self.forward_minibatch_id = 0
        self.backward_minibatch_id = 0
        if self.comm_handler is not None:
            self.comm_handler.set_tensor_shapes(self.tensor_shapes)
            self.comm_handler.start_helper_threads(num_iterations, forward_only=forward_only)
        # the per-minibatch message lists, fixed for the epoch ("ack" and the targets joined the rank maps above)
        self._fwd_recv = [n for n in self.receive_ranks if n != "ack"]
        self._fwd_send = [n for n in self.send_ranks if n != "ack"]
        self._bwd_recv = [n for n in self.send_ranks if self._carries_gradient(n)]
        self._bwd_send = [n for n in self.receive_ranks if self._carries_gradient(n)]
        if self.comm_handler is not None:
            self.comm_handler.gradient_tensor_names = set(self._bwd_recv)

    def train(self, num_iterations):
        self._start(num_iterations, self.training_tensor_shapes, False)
        for m in self.plan.modules:
            m.train()

    def eval(self, num_iterations):
        shapes = self.eval_tensor_shapes
        shapes["ack"] = (1,)
        self.sync_replica_buffers()
        self._start(num_iterations, shapes, True)
        for m in self.plan.modules:
            m.eval()

    def set_loader(self, loader):
        """The stage that owns the data gets an iterable of minibatches, every other stage None
        (runtime/runtime.py:370-374).  The first minibatch is fetched and uploaded here."""
        self.loader_iter = None
        self._feeder = None
        if loader is not None:
            self._feeder = InputFeeder(loader, self.model_type, self.device,
                                       self.training_tensor_dtypes.get("target_length", torch.int),
                                       convert=self._input_convert())
            self.loader_iter = self._feeder

    # ------------------------------------------------------------------ tensor movement
    def receive_tensors_forward(self):
        if self.forward_only and self.tensors:
            self.tensors.pop(0)
        if self._feeder is not None:
            self.tensors.append(self._feeder.next())
            return
        got = {}
        ids = dict(forward_minibatch_id=self.forward_minibatch_id, backward_minibatch_id=self.backward_minibatch_id)
        nbytes = 0
        for name in self._fwd_recv:
            t = self.comm_handler.recv(name, backward=False, **ids)
            got[name] = t
            nbytes += t.element_size() * t.nelement()
        self.forward_stats.stats['receive_tensors_size'] += nbytes
        self.comm_handler.increment_messaging_index(sending=False)
        self.tensors.append(got)

    def send_tensors_forward(self):
        tensors = self.tensors[-1]
        ids = dict(forward_minibatch_id=self.forward_minibatch_id, backward_minibatch_id=self.backward_minibatch_id)
        nbytes = 0
        for name in self._fwd_send:
            t = tensors[name]
            self.comm_handler.send(name, t, backward=False, **ids)
            nbytes += t.element_size() * t.nelement()
        self.forward_stats.stats['send_tensors_size'] += nbytes

    def receive_tensors_backward(self):
        ids = dict(forward_minibatch_id=self.forward_minibatch_id, backward_minibatch_id=self.backward_minibatch_id)
        nbytes = 0
        for name in self._bwd_recv:
            g = self.comm_handler.recv(name, backward=True, **ids)
            self.gradients[name] = g
            nbytes += g.element_size() * g.nelement()
        self.backward_stats.stats['receive_tensors_size'] += nbytes

    def send_tensors_backward(self):
        ids = dict(forward_minibatch_id=self.forward_minibatch_id, backward_minibatch_id=self.backward_minibatch_id)
        nbytes = 0
        for name in self._bwd_send:
            g = self.gradients[name]
            self.comm_handler.send(name, g, backward=True, **ids)
            nbytes += g.element_size() * g.nelement()
        self.backward_stats.stats['send_tensors_size'] += nbytes
        if self.num_ranks_in_previous_stage > 0:
            self.comm_handler.increment_messaging_index(sending=True)

    # ------------------------------------------------------------------ compute
    def _recomputing(self):
        return self.enable_recompute and not self.forward_only and not self.is_criterion

    def run_forward(self, recompute_step=False):
        self.receive_tensors_forward()
        tensors = self.tensors[-1]
        if self._recomputing():
            # no autograd graph and no saved activations: only the stage's inputs stay alive until the
            # backward pass, which runs the forward again (module buffers are put back before that)
            stash = {n: tensors[n] for n in self.plan.inputs if n in tensors}
            for n in self.target_tensor_names:
                if n in tensors:
                    stash[n] = tensors[n]
            state = self._module_replay_state()
            with torch.no_grad():
                self._run_forward(tensors)
            keep = dict(stash)
            keep.update({n: tensors[n] for n in self._fwd_send})
            keep["_replay"] = state
            self.tensors[-1] = keep
        else:
            self._run_forward(tensors)
        if self.comm_handler is not None:
            self.send_tensors_forward()
        if "_replay" in self.tensors[-1]:
            for n in self._fwd_send:                 # sent; only the stage's own inputs wait for the backward pass
                if n not in self.plan.inputs and n not in self.target_tensor_names:
                    self.tensors[-1].pop(n, None)
        if self.verbose_freq > 0 and self.forward_minibatch_id % self.verbose_freq == 0:
            self.forward_stats.print_stats()
        self.forward_stats.reset_stats()
        self.forward_minibatch_id += 1

    def _run_forward(self, tensors):
        self.plan.run(tensors)
        self.output = tensors[self.plan.last_inputs[0]]
        if not self.is_criterion:
            self.loss = 1
        elif self.model_type == TRANSLATION:
            # per-token loss as in runtime/runtime.py:539-542, but divided on the device: reading the
            # token count back here would drain the stream in the middle of every step
            per_batch = tensors[self.plan.last_outputs[0]] * tensors[self.criterion_input_name].size(1)
            self.loss = per_batch / tensors["target_length"][0]
        else:
            self.loss = tensors[self.plan.last_outputs[0]]

    def _module_replay_state(self):
        """What a second forward pass over the same minibatch must see unchanged: module buffers
        (BatchNorm running statistics are updated by a forward pass) and dropout stream positions."""
        bufs = [b.clone() for m in self.plan.modules for b in m.buffers()]
        offs = [(sub, sub.offset) for m in self.plan.modules for sub in m.modules() if hasattr(sub, "offset")
                and isinstance(getattr(sub, "offset"), int)]
        return bufs, offs

    def _replay_forward(self, kept):
        """Recompute: rebuild the minibatch's autograd graph from its stashed inputs, on the weight
        version that is loaded now (the optimizer's `load_old_params` ran just before)."""
        bufs, offs = kept.pop("_replay")
        after = [b.clone() for m in self.plan.modules for b in m.buffers()]
        live = [b for m in self.plan.modules for b in m.buffers()]
        after_offs = [(sub, sub.offset) for (sub, _) in offs]
        for b, saved in zip(live, bufs):
            b.copy_(saved)
        for sub, off in offs:
            sub.offset = off
        tensors = {n: kept[n] for n in kept if n in self.plan.inputs or n in self.target_tensor_names}
        self.plan.run(tensors)
        for b, saved in zip(live, after):
            b.copy_(saved)
        for sub, off in after_offs:
            sub.offset = off
        return tensors

    def run_backward(self):
        self.receive_tensors_backward()
        tensors = self.tensors.pop(0)
        if "_replay" in tensors:
            tensors = self._replay_forward(tensors)

        roots, root_grads = [], []
        for name in self.plan.outputs:
            t = tensors[name]
            if not (torch.is_tensor(t) and t.requires_grad):
                continue
            if name == "loss" and self.loss_scale != 1:
                t = t * self.loss_scale
            roots.append(t)
            root_grads.append(self.gradients.get(name))
        torch.autograd.backward(tuple(roots), grad_tensors=tuple(root_grads))

        for name in self._bwd_send:
            t = tensors[name]
            g = t.grad
            if g is None:
                g = torch.zeros_like(t)          # an input the stage did not use
            self.gradients[name] = g
            t.grad = None
        if self.comm_handler is not None:
            self.send_tensors_backward()
        for name in self._bwd_recv:
            self.gradients.pop(name, None)
        for name in self._bwd_send:
            self.gradients.pop(name, None)
        if self.verbose_freq > 0 and self.backward_minibatch_id % self.verbose_freq == 0:
            self.backward_stats.print_stats()
        self.backward_stats.reset_stats()
        self.backward_minibatch_id += 1

    def num_tokens(self):
        return self.tensors[-1]["target_length"][0].item()

    def run_ack(self):
        """Forward-only runs are clocked by an ack that flows back once per minibatch
        (runtime/runtime.py:629-653), which bounds how far a stage can run ahead of its consumer."""
        if self.rank is None:
            return
        ids = dict(forward_minibatch_id=self.forward_minibatch_id, backward_minibatch_id=self.backward_minibatch_id)
        if self.stage < self.num_stages - 1:
            self.comm_handler.recv("ack", backward=True, **ids)
        if self.stage > 0:
            ack = torch.zeros(self.tensor_shapes["ack"], dtype=torch.int64, device=self.device)
            self.comm_handler.send("ack", ack, backward=True, **ids)
            self.comm_handler.increment_messaging_index(sending=True)
        self.backward_minibatch_id += 1

    def wait(self):
        if self.comm_handler is not None:
            self.comm_handler.wait()

    def num_iterations(self, loader_size):
        """Minibatches this stage sees per epoch: the loader's count scaled by the replica ratio
        (runtime/runtime.py:659-671)."""
        if not self.stage:
            return loader_size
        total = loader_size * self.num_ranks_in_first_stage
        if total % self.num_ranks_in_stage:
            raise AssertionError("%d minibatches do not divide over %d replicas" % (total, self.num_ranks_in_stage))
        return total // self.num_ranks_in_stage

    def get_adjusted_learning_rate(self, base_lr):
        """A stage with R_s replicas sees R_s/R_0 times the per-replica batch of stage 0
        (runtime/runtime.py:673-680)."""
        if self.stage == 0:
            return base_lr
        return float(base_lr) * float(self.num_ranks_in_stage) / float(self.num_ranks_in_first_stage)


class GradientAverager:
    """Sums a stage's flat fp32 gradient arena over its replicas; returns the factor that turns the sum into
    the mean (the optimizer folds it into the gradient scale of its fused kernel).  Stands where the
    reference wraps the stage in DistributedDataParallel (runtime/runtime.py:232-262) and, like it, reduces in
    buckets while the backward pass is still running:

    * the arena is cut into contiguous buckets of about `bucket_bytes`; parameters are laid out in forward order,
      so the backward pass finishes the buckets from the last to the first;
    * every native layer announces a gradient write just before it enqueues the writing kernel; when a bucket's last
      parameter has been announced and the NEXT announcement arrives (so the writing kernel is in the stream), an
      event is recorded and the bucket's all-reduce is issued on a side stream behind that event;
    * `__call__` (from the optimizer's step) issues whatever is left and makes the compute stream wait for the
      side stream - only the last bucket's reduction is exposed.

    The first minibatch runs as one blocking all-reduce while the announcements are counted: a parameter that is
    written more than once per backward pass (shared between two layers of the stage) would be reduced too early,
    so a stage with such a parameter keeps the blocking form.  Gradient accumulation over several minibatches
    (`update_interval` > 1) keeps it as well."""

    def __init__(self, group, world, bucket_bytes=32 << 20):
        self.group, self.world = group, world
        self.bucket_bytes = bucket_bytes
        self.opt = None
        self.mode = "learn"            # learn -> overlap | blocking
        self.counts = {}
        self.stream = None

    # -- set-up ------------------------------------------------------------------------------------------
    def bind(self, optimizer):
        """Called by the optimizer once its arena exists."""
        self.opt = optimizer
        if self.group is None or optimizer.update_interval != 1 or optimizer.grad_arena.device.type != "cuda":
            self.mode = "blocking"
            return
        for p in optimizer.master_parameters:
            p._pd_grad_hook = self._announce

    def _plan(self):
        opt = self.opt
        self.bucket_of, self.buckets = {}, []
        lo, members = None, []
        for p, (off, span) in zip(opt.master_parameters, opt._offsets):
            if lo is None:
                lo = off
            members.append(p)
            end = (off + span + 63) // 64 * 64
            if (end - lo) * 4 >= self.bucket_bytes:
                self.buckets.append({"lo": lo, "hi": end, "members": members})
                lo, members = None, []
        if members:
            end = (opt._offsets[-1][0] + opt._offsets[-1][1] + 63) // 64 * 64
            self.buckets.append({"lo": lo, "hi": end, "members": members})
        for b in self.buckets:
            for p in b["members"]:
                self.bucket_of[id(p)] = b
        self.stream = torch.cuda.Stream(device=opt.grad_arena.device)
        self._reset()

    def _reset(self):
        for b in self.buckets:
            b["left"] = len(b["members"])
            b["sent"] = False
        self.previous = None

    # -- backward pass -----------------------------------------------------------------------------------
    def _announce(self, param):
        if self.mode == "learn":
            self.counts[id(param)] = self.counts.get(id(param), 0) + 1
            return
        if self.mode != "overlap":
            return
        prev, self.previous = self.previous, param
        if prev is not None:
            b = self.bucket_of[id(prev)]
            b["left"] -= 1
            if b["left"] == 0:
                self._send(b)

    def _send(self, b):
        if b["sent"]:
            return
        b["sent"] = True
        arena = self.opt.grad_arena
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(arena.device))
        self.stream.wait_event(ev)
        with torch.cuda.stream(self.stream):
            dist.all_reduce(arena[b["lo"]:b["hi"]], op=dist.ReduceOp.SUM, group=self.group)

    # -- optimizer step ----------------------------------------------------------------------------------
    def __call__(self, grad_arena):
        if self.group is None:
            return 1.0
        if self.mode == "overlap":
            for b in self.buckets:
                self._send(b)
            done = torch.cuda.Event()
            done.record(self.stream)
            torch.cuda.current_stream(grad_arena.device).wait_event(done)
            self._reset()
            return 1.0 / self.world
        dist.all_reduce(grad_arena, op=dist.ReduceOp.SUM, group=self.group)
        if self.mode == "learn" and self.opt is None:
            self.mode = "blocking"         # used without an arena (no optimizer bound): nothing to bucket
        if self.mode == "learn":
            once = all(c == 1 for c in self.counts.values())
            # every replica must take the same decision: they all run the same stage code, but be explicit
            flag = torch.tensor([1 if once else 0], device=grad_arena.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            self.mode = "overlap" if int(flag.item()) == 1 else "blocking"
            if self.mode == "overlap":
                self._plan()
        return 1.0 / self.world
