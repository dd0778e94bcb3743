"""Stage runtime with the interface of the reference's runtime/runtime.py:44-680.

`StageRuntime` keeps the constructor signature, methods and attributes that
main_with_runtime.py uses (`train`, `eval`, `set_loader`, `run_forward`,
`run_backward`, `run_ack`, `wait`, `num_iterations`,
`get_adjusted_learning_rate`, `state_dict`, `load_state_dict`, `modules`,
`parameters`, `zero_grad`, `stage`, `num_stages`, `num_ranks`,
`num_warmup_minibatches`, `rank_in_stage`, `num_ranks_in_first_stage`,
`master_parameters`, `model_parameters`, `output`, `target`, `loss`) and the
stage / rank / warm-up arithmetic of its `initialize` (:80-291).  Underneath,
the stage's leaf modules are swapped for CUDA-native ones (layers.nativize),
boundary tensors move over NVLink peer channels instead of gloo, and a
replicated stage averages its flat gradient arena with one NCCL all-reduce per
optimizer step instead of DistributedDataParallel.
"""
import collections
import itertools
import os

import torch
import torch.distributed as dist

from . import communication
from . import layers
from . import runtime_utilities

IMAGE_CLASSIFICATION = "image_classification"
TRANSLATION = "translation"
SPEECH_TO_TEXT = "speech_to_text"


class ModulesWithDependencies:
    def __init__(self, modules_with_dependencies):
        self._modules = []
        self._all_input_names = []
        self._all_output_names = []
        for (module, input_names, output_names) in modules_with_dependencies:
            self._modules.append(module)
            self._all_input_names.append(input_names)
            self._all_output_names.append(output_names)

    def modules(self):
        return self._modules

    def all_input_names(self):
        return self._all_input_names

    def all_output_names(self):
        return self._all_output_names

    def is_input_tensor(self, tensor_name):
        return any(tensor_name in names for names in self._all_input_names)


def stage_assignment(num_modules, configuration_maps, rank):
    """Pure arithmetic of runtime/runtime.py:129-175: which modules, stage, replica index and
    warm-up depth a rank gets.  Returns a dict; no side effects (used by the CPU tests)."""
    module_to_stage_map = configuration_maps['module_to_stage_map']
    stage_to_rank_map = configuration_maps['stage_to_rank_map']
    stage_to_depth_map = configuration_maps.get('stage_to_depth_map')
    assert len(module_to_stage_map) == num_modules
    stage_to_module_map = collections.defaultdict(list)
    for module in range(len(module_to_stage_map)):
        stage_to_module_map[module_to_stage_map[module]].append(module)
    rank_to_stage_map = {}
    for stage in stage_to_rank_map:
        for r in stage_to_rank_map[stage]:
            rank_to_stage_map[r] = stage
    assert 0 <= rank < len(rank_to_stage_map)
    out = {}
    out["num_ranks"] = len(rank_to_stage_map)
    out["num_stages"] = len(stage_to_module_map)
    stage = rank_to_stage_map[rank]
    out["stage"] = stage
    out["rank_in_stage"] = stage_to_rank_map[stage].index(rank)
    out["num_ranks_in_stage"] = len(stage_to_rank_map[stage])
    out["num_ranks_in_first_stage"] = len(stage_to_rank_map[0])
    out["ranks_in_previous_stage"] = list(stage_to_rank_map[stage - 1]) if stage > 0 else []
    out["ranks_in_next_stage"] = list(stage_to_rank_map[stage + 1]) if stage < out["num_stages"] - 1 else []
    out["modules"] = stage_to_module_map[stage]
    out["is_criterion"] = stage == out["num_stages"] - 1
    if stage_to_depth_map is not None:
        out["num_warmup_minibatches"] = stage_to_depth_map[str(stage)]
    else:
        w = out["num_ranks"] - 1
        for i in range(stage):
            w -= len(stage_to_rank_map[i])
        out["num_warmup_minibatches"] = w // out["num_ranks_in_stage"]
    return out


class StageRuntime:
    def __init__(self, model, distributed_backend, fp16, loss_scale,
                 training_tensor_shapes, eval_tensor_shapes,
                 training_tensor_dtypes, inputs_module_destinations,
                 target_tensor_names, configuration_maps, master_addr,
                 rank, local_rank, num_ranks_in_server, verbose_freq,
                 model_type, enable_recompute=False, device=None, native=True):
        """Arguments up to `enable_recompute` are the reference's (runtime/runtime.py:45-50);
        `fp16=True` selects 16-bit compute, which on this hardware is bf16 with fp32 master
        weights inside the optimizer.  `device` / `native` exist for the host-logic tests
        (CPU ranks with unswapped modules); the defaults are the product path: CUDA device
        `local_rank`, native kernels, and an error if either is unavailable."""
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
        self.native = native
        if device is None:
            if not torch.cuda.is_available():
                raise RuntimeError("pipedream_b200.StageRuntime needs a CUDA device (there is no CPU path)")
            device = torch.device("cuda", local_rank if local_rank is not None else 0)
        self.device = torch.device(device)
        if self.native:
            if self.device.type != "cuda":
                raise RuntimeError("native kernels need a CUDA device")
            from . import _lib
            _lib.load()       # fail now, loudly, if the CUDA library was not built
            _lib.call("pd_device_ok")

        self.initialize(model, inputs_module_destinations, configuration_maps,
                        master_addr, rank, local_rank, num_ranks_in_server)

        self.verbose_freq = verbose_freq
        self.forward_only = False
        self.forward_stats = runtime_utilities.RuntimeStats(forward=True)
        self.backward_stats = runtime_utilities.RuntimeStats(forward=False)
        # Parsed and stored, never acted on - as in the reference (runtime/runtime.py:72-78).
        self.enable_recompute = enable_recompute
        if rank == num_ranks_in_server - 1:
            self.enable_recompute = False

    # ------------------------------------------------------------------ set-up
    def initialize(self, model, inputs_module_destinations, configuration_maps,
                   master_addr, rank, local_rank, num_ranks_in_server):
        self.send_ranks = {}
        self.receive_ranks = {}
        self.rank = rank
        self.local_rank = local_rank
        self.stage = None
        self.tensor_tags = {}
        self.forward_minibatch_id = 0
        self.backward_minibatch_id = 0
        self.criterion_input_name = str(model[-1][1][0])

        tensor_tag = 1
        for (_, input_tensors, output_tensors) in model:
            for input_tensor in input_tensors:
                if input_tensor not in self.tensor_tags:
                    self.tensor_tags[input_tensor] = tensor_tag
                    tensor_tag += 1
            for output_tensor in output_tensors:
                if output_tensor not in self.tensor_tags:
                    self.tensor_tags[output_tensor] = tensor_tag
                    tensor_tag += 1
        for target_tensor_name in sorted(self.target_tensor_names):
            self.tensor_tags[target_tensor_name] = tensor_tag
            tensor_tag += 1
        self.tensor_tags["ack"] = tensor_tag
        tensor_tag += 1

        module_to_stage_map = configuration_maps['module_to_stage_map']
        stage_to_rank_map = configuration_maps['stage_to_rank_map']

        if module_to_stage_map is None:
            # Single process: every module, no communication (runtime/runtime.py:113-127).
            assert self.rank is None
            self.modules_with_dependencies = ModulesWithDependencies(model)
            self.is_criterion = True
            self.rank_in_stage = 0
            self.num_ranks = 1
            self.num_ranks_in_first_stage = 1
            self.num_ranks_in_previous_stage = 0
            self.num_ranks_in_next_stage = 0
            self.num_stages = 1
            self.num_ranks_in_stage = 1
            self.num_warmup_minibatches = 0
            self.comm_handler = None
            self.ranks_in_previous_stage = []
            self.ranks_in_next_stage = []
        else:
            assert self.rank is not None
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
            self.modules_with_dependencies = ModulesWithDependencies([model[m] for m in a["modules"]])
            self.is_criterion = a["is_criterion"]
            self.num_warmup_minibatches = a["num_warmup_minibatches"]

            # fixed port of the reference (runtime/runtime.py:181); overridable for concurrent jobs
            master_port = int(os.environ.get("PIPEDREAM_MASTER_PORT", "12345"))
            self.comm_handler = communication.CommunicationHandler(
                master_addr=master_addr, master_port=master_port, rank=self.rank,
                local_rank=self.local_rank, num_ranks_in_server=num_ranks_in_server,
                world_size=self.num_ranks, fp16=self.fp16, backend=self.distributed_backend)

            # Producer / consumer ranks of every tensor that crosses a stage boundary.
            for i in range(len(model)):
                for j in range(i + 1, len(model)):
                    for tensor_name in model[i][2]:
                        if tensor_name in model[j][1]:
                            if module_to_stage_map[i] == module_to_stage_map[j]:
                                continue
                            if module_to_stage_map[j] == self.stage:
                                self.receive_ranks[tensor_name] = stage_to_rank_map[module_to_stage_map[i]]
                            if module_to_stage_map[i] == self.stage:
                                self.send_ranks[tensor_name] = stage_to_rank_map[module_to_stage_map[j]]
            # Model inputs needed by a later stage are forwarded hop by hop.
            for model_inputs in inputs_module_destinations.keys():
                destination_stage = module_to_stage_map[inputs_module_destinations[model_inputs]]
                if destination_stage > self.stage:
                    self.send_ranks[model_inputs] = self.ranks_in_next_stage
                if 0 < self.stage <= destination_stage:
                    self.receive_ranks[model_inputs] = self.ranks_in_previous_stage
                if destination_stage > 0:
                    if model_inputs not in self.tensor_tags:
                        self.tensor_tags[model_inputs] = tensor_tag
                        tensor_tag += 1

        modules = self.modules_with_dependencies.modules()
        compute_dtype = torch.bfloat16 if self.fp16 else torch.float32
        for i in range(len(modules)):
            modules[i] = modules[i].to(self.device)
            if self.fp16:
                modules[i] = modules[i].to(compute_dtype)
            if self.native:
                modules[i] = layers.nativize(modules[i])
        self.compute_dtype = compute_dtype

        # Replicated stage: one process group per stage, created in the same order everywhere.
        self.stage_group = None
        if stage_to_rank_map is not None and self.distributed_backend != communication.LOCAL:
            groups = []
            for stage in range(self.num_stages):
                ranks = stage_to_rank_map[stage]
                groups.append(dist.new_group(ranks=ranks) if len(ranks) > 1 else None)
            self.stage_group = groups[self.stage]
        if self.num_ranks_in_stage > 1:
            num_parameters = sum(p.numel() for p in self.parameters())
            print("Replicating stage: ranks=%d, module_size=%.3f" % (
                self.num_ranks_in_stage, 4. * num_parameters))
            sync = self._make_grad_sync()
            for m in modules:
                m._pd_grad_sync = sync

        # 16-bit master weights live inside the optimizer's arena, so the two lists of the
        # reference (apex prep_param_lists, runtime/runtime.py:268-276) collapse into one.
        self.master_parameters = list(self.parameters())
        self.model_parameters = None

        if self.comm_handler is not None:
            self.comm_handler.variable_shapes = (self.model_type == TRANSLATION)
            self.comm_handler.initialize(
                self.receive_ranks, self.send_ranks, self.tensor_tags,
                self.target_tensor_names, self.training_tensor_dtypes,
                self.rank_in_stage, self.num_ranks_in_stage,
                self.ranks_in_previous_stage, self.ranks_in_next_stage)

    def _make_grad_sync(self):
        """Average the flat gradient arena over the replicas of this stage (the reference wraps
        the stage in DistributedDataParallel, runtime/runtime.py:258-262)."""
        group, world = self.stage_group, self.num_ranks_in_stage

        def sync(grad_arena):
            """Sums the arena over the replicas; returns the factor that turns the sum into the mean
            (the optimizer folds it into the gradient scale of its fused kernel)."""
            if group is None:
                return 1.0
            dist.all_reduce(grad_arena, op=dist.ReduceOp.SUM, group=group)
            return 1.0 / world
        return sync

    # ------------------------------------------------------------------ accessors
    @property
    def target(self):
        return self.tensors[-1]["target"]

    def modules(self):
        return self.modules_with_dependencies.modules()

    def parameters(self):
        return itertools.chain(*[m.parameters() for m in self.modules_with_dependencies.modules()])

    def state_dict(self):
        state_dict = collections.OrderedDict()
        for i, module in enumerate(self.modules_with_dependencies.modules()):
            state_dict["module%d" % i] = module.state_dict()
        return state_dict

    def load_state_dict(self, state_dict):
        for i, module in enumerate(self.modules_with_dependencies.modules()):
            module.load_state_dict(state_dict["module%d" % i])

    def cuda(self):
        modules = self.modules_with_dependencies.modules()
        for i in range(len(modules)):
            modules[i] = modules[i].to(self.device)

    def zero_grad(self):
        for p in self.parameters():
            p._pd_acc = False
            if p.grad is not None and p.grad is not getattr(p, "_pd_grad", None):
                p.grad = None

    # ------------------------------------------------------------------ epoch control
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

    def train(self, num_iterations):
        self._start(num_iterations, self.training_tensor_shapes, False)
        for m in self.modules_with_dependencies.modules():
            m.train()

    def eval(self, num_iterations):
        shapes = self.eval_tensor_shapes
        shapes["ack"] = (1,)
        self._start(num_iterations, shapes, True)
        for m in self.modules_with_dependencies.modules():
            m.eval()

    def set_loader(self, loader):
        self.loader_iter = iter(loader) if loader is not None else None

    # ------------------------------------------------------------------ tensor movement
    def _to_device(self, t):
        return t.to(self.device, non_blocking=True)

    def receive_tensors_forward(self):
        if self.forward_only and len(self.tensors) > 0:
            self.tensors.pop(0)
        self.tensors.append({})
        if self.loader_iter is not None:
            input = next(self.loader_iter)
            if self.model_type == TRANSLATION:
                (input, target) = input
                src, src_length = input
                tgt, tgt_length = target
                self.tensors[-1]["input0"] = self._to_device(src)
                self.tensors[-1]["input1"] = self._to_device(torch.as_tensor(src_length, dtype=torch.int64))
                self.tensors[-1]["input2"] = self._to_device(tgt[:-1])
                self.tensors[-1]["target"] = self._to_device(tgt[1:]).contiguous().view(-1)
                self.tensors[-1]["target_length"] = self._to_device(torch.tensor(
                    [int(sum(torch.as_tensor(tgt_length, dtype=torch.int64) - 1))],
                    dtype=self.training_tensor_dtypes.get("target_length", torch.int)))
            elif self.model_type == IMAGE_CLASSIFICATION:
                (input, target) = input
                if self.fp16 and not self.native:
                    input = input.to(self.compute_dtype)     # runtime/runtime.py:397-398 (native
                    # stages convert inside their first kernel instead)
                self.tensors[-1]["input0"] = self._to_device(input)
                self.tensors[-1]["target"] = self._to_device(target)
            else:
                raise NotImplementedError("model_type %r is not supported" % (self.model_type,))
        else:
            for input_name in self.receive_ranks:
                if input_name == "ack":
                    continue
                self.tensors[-1][input_name] = self.comm_handler.recv(
                    input_name, forward_minibatch_id=self.forward_minibatch_id,
                    backward_minibatch_id=self.backward_minibatch_id, backward=False)
                self.forward_stats.stats['receive_tensors_size'] += (
                    self.tensors[-1][input_name].element_size() * self.tensors[-1][input_name].nelement())
            self.comm_handler.increment_messaging_index(sending=False)

    def send_tensors_forward(self):
        for output_name in self.send_ranks:
            if output_name == "ack":
                continue
            self.comm_handler.send(
                output_name, self.tensors[-1][output_name],
                forward_minibatch_id=self.forward_minibatch_id,
                backward_minibatch_id=self.backward_minibatch_id, backward=False)
            self.forward_stats.stats['send_tensors_size'] += (
                self.tensors[-1][output_name].element_size() * self.tensors[-1][output_name].nelement())

    def receive_tensors_backward(self):
        for output_name in self.send_ranks:
            if output_name in self.target_tensor_names:
                continue
            self.gradients[output_name] = self.comm_handler.recv(
                output_name, forward_minibatch_id=self.forward_minibatch_id,
                backward_minibatch_id=self.backward_minibatch_id, backward=True)
            self.backward_stats.stats['receive_tensors_size'] += (
                self.gradients[output_name].element_size() * self.gradients[output_name].nelement())

    def send_tensors_backward(self):
        for input_name in self.receive_ranks:
            if input_name in self.target_tensor_names:
                continue
            self.comm_handler.send(
                input_name, self.gradients[input_name],
                forward_minibatch_id=self.forward_minibatch_id,
                backward_minibatch_id=self.backward_minibatch_id, backward=True)
            self.backward_stats.stats['send_tensors_size'] += (
                self.gradients[input_name].element_size() * self.gradients[input_name].nelement())
        if self.num_ranks_in_previous_stage > 0:
            self.comm_handler.increment_messaging_index(sending=True)

    # ------------------------------------------------------------------ compute
    def run_forward(self, recompute_step=False):
        self.receive_tensors_forward()
        tensors = self.tensors[-1]
        self._run_forward(tensors)
        self.send_tensors_forward()
        if self.verbose_freq > 0 and self.forward_minibatch_id % self.verbose_freq == 0:
            self.forward_stats.print_stats()
        self.forward_stats.reset_stats()
        self.forward_minibatch_id += 1

    def _run_forward(self, tensors):
        modules = self.modules_with_dependencies.modules()
        all_input_names = self.modules_with_dependencies.all_input_names()
        all_output_names = self.modules_with_dependencies.all_output_names()
        for i, (module, input_names, output_names) in enumerate(zip(modules, all_input_names, all_output_names)):
            if i == (len(modules) - 1) and self.is_criterion:
                module_outputs = [module(tensors[input_name], tensors["target"]) for input_name in input_names]
                module_outputs = [sum(module_outputs)]
            else:
                module_outputs = module(*[tensors[input_name] for input_name in input_names])
                if not isinstance(module_outputs, tuple):
                    module_outputs = (module_outputs,)
                module_outputs = list(module_outputs)
            for (output_name, module_output) in zip(output_names, module_outputs):
                tensors[output_name] = module_output

        self.output = tensors[input_names[0]]
        if self.is_criterion and self.model_type == TRANSLATION:
            # per-token loss as in runtime/runtime.py:539-542, but divided on the device: reading the
            # token count back here would drain the stream in the middle of every step
            loss_per_batch = tensors[output_names[0]] * tensors[self.criterion_input_name].size(1)
            self.loss = loss_per_batch / tensors["target_length"][0]
        elif self.is_criterion:
            self.loss = tensors[output_names[0]]
        else:
            self.loss = 1

    def run_backward(self):
        self.receive_tensors_backward()
        inputs, outputs = {}, {}
        input_gradients, output_gradients = {}, {}
        all_input_names_set, all_output_names_set = set(), set()

        modules = self.modules_with_dependencies.modules()
        all_input_names = self.modules_with_dependencies.all_input_names()
        all_output_names = self.modules_with_dependencies.all_output_names()
        for (input_names, output_names) in zip(all_input_names, all_output_names):
            all_input_names_set.update(input_names)
            all_output_names_set.update(output_names)

        tensors = self.tensors.pop(0)
        # Stage outputs are tensors no module of this stage consumes; stage inputs are tensors
        # no module of this stage produces (runtime/runtime.py:577-592).
        for (module, input_names, output_names) in zip(reversed(modules), reversed(all_input_names),
                                                       reversed(all_output_names)):
            for output_name in output_names:
                if output_name not in all_input_names_set:
                    output_gradients[output_name] = self.gradients.get(output_name)
                    if tensors[output_name].requires_grad:
                        outputs[output_name] = tensors[output_name]
            for input_name in input_names:
                if input_name not in all_output_names_set:
                    inputs[input_name] = tensors[input_name]

        def hook_wrapper(input_name):
            def hook(input_gradient):
                input_gradients[input_name] = input_gradient
            return hook

        for input_name in inputs:
            if input_name not in ("input0", "input1", "input2") and inputs[input_name].requires_grad:
                inputs[input_name].register_hook(hook_wrapper(input_name))

        if "loss" in outputs and self.loss_scale != 1:
            outputs["loss"] = outputs["loss"] * self.loss_scale

        torch.autograd.backward(tuple(outputs[name] for name in outputs),
                                grad_tensors=tuple(output_gradients[name] for name in outputs))

        for input_name in inputs:
            if not inputs[input_name].requires_grad:
                self.gradients[input_name] = inputs[input_name]
                continue
            if input_name not in ("input0", "input1", "input2", "input"):
                self.gradients[input_name] = input_gradients[input_name]

        self.send_tensors_backward()
        if self.verbose_freq > 0 and self.backward_minibatch_id % self.verbose_freq == 0:
            self.backward_stats.print_stats()
        self.backward_stats.reset_stats()
        self.backward_minibatch_id += 1

    def num_tokens(self):
        return self.tensors[-1]["target_length"][0].item()

    def run_ack(self):
        """Forward-only clock: an ack flows backwards once per minibatch (runtime/runtime.py:629-653)."""
        if self.rank is None:
            return
        if self.stage < (self.num_stages - 1):
            self.comm_handler.recv("ack", forward_minibatch_id=self.forward_minibatch_id,
                                   backward_minibatch_id=self.backward_minibatch_id, backward=True)
        if self.stage > 0:
            self.comm_handler.send("ack", torch.zeros(self.tensor_shapes["ack"], dtype=torch.int64,
                                                      device=self.device),
                                   forward_minibatch_id=self.forward_minibatch_id,
                                   backward_minibatch_id=self.backward_minibatch_id, backward=True)
            self.comm_handler.increment_messaging_index(sending=True)
        self.backward_minibatch_id += 1

    def wait(self):
        if self.comm_handler is not None:
            self.comm_handler.wait()

    def num_iterations(self, loader_size):
        """Minibatches this stage sees per epoch (runtime/runtime.py:659-671)."""
        if self.stage == 0 or self.stage is None:
            return loader_size
        num_iterations = loader_size * self.num_ranks_in_first_stage
        assert num_iterations % self.num_ranks_in_stage == 0
        return num_iterations // self.num_ranks_in_stage

    def get_adjusted_learning_rate(self, base_lr):
        """Per-stage learning-rate scale (runtime/runtime.py:673-680)."""
        if self.stage == 0:
            return base_lr
        return float(base_lr) * float(self.num_ranks_in_stage) / float(self.num_ranks_in_first_stage)
