"""Weight stashing over an in-HBM ring of weight versions.

Mirrors the interface of the reference wrapper (runtime/optimizer.py:19-164:
`OptimizerWithWeightStashing`, `Version`, `load_old_params`, `load_new_params`,
`zero_grad`, `step`, attributes `queue`, `latest_version`, `current_version`,
`num_versions`), but not its mechanism.  The reference keeps a deque of cloned
state_dicts and copies a full model three times per minibatch; here all
parameters of the stage live in one flat arena with `num_versions` slots:

    slot(v) = v mod num_versions

`load_old_params` / `load_new_params` re-point `param.data` at another slot
(no copy), and `step` is one fused kernel launch that reads the gradient arena,
the newest weights (fp32 master when the compute copy is bf16) and the
optimizer state, and writes version latest+1 into the slot of the oldest
version.  The forward pass of a minibatch captures aliases of the slot that is
current at that time, so its delayed backward pass reads exactly the weights
its forward pass used.
"""
import ctypes
import time

import torch

from . import _lib
from ._lib import call
from . import functional as pf


class Version:
    """Same value type as runtime/optimizer.py:9-17."""

    def __init__(self, version=0):
        self.version = version

    def __repr__(self):
        return "v%d" % self.version

    def __eq__(self, other):
        return isinstance(other, Version) and other.version == self.version

    def __hash__(self):
        return hash(self.version)

    def incr(self):
        return Version(version=self.version + 1)


class VersionRing:
    """Pure index arithmetic of the version ring (no device memory).

    Reproduces which version the reference's deque(maxlen=num_versions) holds at
    its two ends (runtime/optimizer.py:58-62,110-116,157-159): the deque starts
    with num_versions copies of v0 and every step appends latest+1.
    """

    def __init__(self, num_versions):
        assert num_versions >= 1
        self.num_versions = num_versions
        self.latest = 0

    def slot(self, version):
        return version % self.num_versions

    def oldest(self):
        return max(0, self.latest - self.num_versions + 1)

    def newest(self):
        return self.latest

    def versions(self):
        """Version tags of the deque entries, oldest first (length num_versions)."""
        n, l = self.num_versions, self.latest
        return [max(0, l - n + 1 + i) for i in range(n)]

    def advance(self):
        """A step was taken: returns (read_slot, write_slot) of the fused update."""
        read = self.slot(self.latest)
        self.latest += 1
        return read, self.slot(self.latest)


def _align(n, a):
    return (n + a - 1) // a * a


class OptimizerWithWeightStashing:
    """Wrapper that adds weight stashing to SGD / Adam (see module docstring).

    Arguments follow runtime/optimizer.py:28-30.  `model_parameters` is accepted
    for signature compatibility; 16-bit master weights are kept inside the arena.
    """

    _SUPPORTED = ("SGD", "Adam")

    def __init__(self, optim_name, modules, master_parameters, model_parameters,
                 loss_scale, num_versions, verbose_freq=0, macrobatch=False,
                 **optimizer_args):
        # (an argument of this implementation, not the reference's; taken out before the rest reaches torch.optim)
        update_interval = optimizer_args.pop("update_interval", None)
        if optim_name not in self._SUPPORTED:
            raise ValueError("optimizer %r is not supported (SGD, Adam)" % optim_name)
        self.optim_name = optim_name
        self.modules = modules
        self.master_parameters = list(master_parameters)
        self.model_parameters = model_parameters
        self.loss_scale = loss_scale
        if macrobatch:
            num_versions = min(2, num_versions)
        self.num_versions = num_versions
        # The torch optimizer object only holds hyper-parameters (param_groups is
        # what the driver script mutates to set the learning rate) and exposes the
        # optimizer state for checkpoints; its step() is never called.
        self.base_optimizer = getattr(torch.optim, optim_name)(self.master_parameters, **optimizer_args)
        self.latest_version = Version()
        self.current_version = Version()
        self.verbose_freq = verbose_freq
        self.batch_counter = 0
        # The reference ties the accumulation length to the (capped) version count: a macrobatch is
        # `num_versions` <= 2 minibatches (runtime/optimizer.py:36-52).  `update_interval` (an extension, not in the
        # reference's signature) sets it independently, e.g. 64 microbatches of 8 sequences for a global batch of
        # 512 with two weight versions; gradients accumulate in the fp32 arena and are scaled by 1 / interval.
        self.update_interval = self.num_versions if macrobatch else 1
        if update_interval is not None:
            if not macrobatch or int(update_interval) < 1:
                raise ValueError("update_interval needs macrobatch=True and a positive value")
            self.update_interval = int(update_interval)
        self.trace = []           # (event, version) tuples; tests compare it with the reference's
        self._steps_taken = 0
        self._grad_sync = None    # set by StageRuntime for replicated stages
        for m in modules:
            sync = getattr(m, "_pd_grad_sync", None)
            if sync is not None:
                self._grad_sync = sync
        self._build_arena()
        self.initialize_queue()
        if self._grad_sync is not None and hasattr(self._grad_sync, "bind"):
            self._grad_sync.bind(self)         # bucketed, backward-overlapped reduction needs the arena layout
        for m in modules:
            rt = getattr(m, "_pd_runtime", None)
            rt = rt() if rt is not None else None
            if rt is not None:
                rt.attach_optimizer(self)      # StageRuntime.load_state_dict re-seeds the ring through this

    def __getattr__(self, key):
        """Relay unknown attributes to the torch optimizer (param_groups, state_dict, ...)."""
        if key == "base_optimizer":
            raise AttributeError(key)
        return getattr(self.base_optimizer, key)

    # ------------------------------------------------------------------ arena
    def _build_arena(self):
        params = self.master_parameters
        if not params:
            raise ValueError("stage has no parameters")
        dev = params[0].device
        if dev.type != "cuda":
            raise _lib.PipedreamB200Error("OptimizerWithWeightStashing needs CUDA parameters (no CPU path)")
        dtype = params[0].dtype
        for p in params:
            if p.dtype != dtype or p.device != dev:
                raise ValueError("all parameters of a stage must share dtype and device")
        self.dtype = dtype
        self.device = dev
        offsets, total = [], 0
        for p in params:
            d = p.data
            span = 1 + sum((s - 1) * st for s, st in zip(d.shape, d.stride())) if d.numel() else 0
            offsets.append((total, span))
            total = _align(total + span, 64)
        self.numel = total
        self.slot_stride = _align(total, 64)
        V = self.num_versions
        self.arena = torch.zeros(V, self.slot_stride, dtype=dtype, device=dev)
        self.grad_arena = torch.zeros(self.slot_stride, dtype=torch.float32, device=dev)
        self.master = torch.zeros(self.slot_stride, dtype=torch.float32, device=dev) \
            if dtype != torch.float32 else None
        self.state_a = torch.zeros(self.slot_stride, dtype=torch.float32, device=dev)   # momentum / exp_avg
        self.state_b = torch.zeros(self.slot_stride, dtype=torch.float32, device=dev) \
            if self.optim_name == "Adam" else None
        self._offsets = offsets
        self._views = []      # per slot: list of parameter views
        for s in range(V):
            views = []
            for p, (off, _) in zip(params, offsets):
                views.append(self.arena[s].as_strided(p.data.shape, p.data.stride(), s * self.slot_stride + off))
            self._views.append(views)
        # seed slot 0 with the current weights, then alias the parameters onto it
        for p, v, (off, _) in zip(params, self._views[0], offsets):
            v.copy_(p.data)
            if self.master is not None:
                self.master.as_strided(p.data.shape, p.data.stride(), off).copy_(p.data)
            g = self.grad_arena.as_strided(p.data.shape, p.data.stride(), off)
            p._pd_grad = g
            p._pd_acc = False
            p.grad = g if dtype == torch.float32 else None
        self._point_params(0)

    def _point_params(self, slot):
        for p, v in zip(self.master_parameters, self._views[slot]):
            p.data = v
        self._current_slot = slot

    # ------------------------------------------------------------------ queue
    def initialize_queue(self):
        """All num_versions entries start as copies of the current weights, tagged v0
        (runtime/optimizer.py:58-62).  Only slot 0 needs data: the other slots are
        written before they are first read."""
        self.ring = VersionRing(self.num_versions)
        self.ring.latest = self.latest_version.version
        self._valid_slots = {self.ring.slot(self.latest_version.version)}

    @property
    def queue(self):
        """[(parameter views, Version)] oldest first, like the reference's deque."""
        out = []
        for v in self.ring.versions():
            out.append((self._views[self.ring.slot(v)], Version(v)))
        return out

    def get_params(self, clone):
        views = self._views[self._current_slot]
        if clone:
            return [v.clone() for v in views], self.latest_version
        return views, self.latest_version

    def set_params(self, state_dicts, version):
        """Makes `version` the one the modules compute with (runtime/optimizer.py:96-108).  The reference copies
        `state_dicts` into the modules; here the version number alone selects a slot of the ring and the
        parameters are re-pointed at it, so `state_dicts` (what `get_params` or `queue` handed out) is not read."""
        self._point_params(self.ring.slot(version.version))
        self.current_version = version

    def load_old_params(self):
        if self.num_versions > 1:
            v = Version(self.ring.oldest())
            self.set_params(self._views[self.ring.slot(v.version)], v)
        self.trace.append(("load_old", self.current_version.version))

    def load_new_params(self):
        if self.num_versions > 1:
            v = Version(self.ring.newest())
            self.set_params(self._views[self.ring.slot(v.version)], v)
        self.trace.append(("load_new", self.current_version.version))

    # ------------------------------------------------------------------ step
    def zero_grad(self):
        if self.batch_counter % self.update_interval == 0:
            for p in self.master_parameters:
                p._pd_acc = False
                if getattr(p, "_pd_native", False):
                    continue          # the first kernel write after this overwrites the buffer
                # parameters of modules that were not swapped: autograd accumulates into .grad
                if p.grad is p._pd_grad:
                    p._pd_grad.zero_()
                    p._pd_foreign_seen = False
                else:
                    p.grad = None

    def _collect_foreign_grads(self):
        """Parameters of modules that were not swapped get their gradient from autograd."""
        for p in self.master_parameters:
            if getattr(p, "_pd_native", False):
                continue
            g = p.grad
            if g is None:
                continue
            if g is not p._pd_grad:
                p._pd_grad.copy_(g)
            p._pd_acc = True

    def _segments(self):
        """Contiguous arena ranges of parameters that received a gradient."""
        segs = []
        for p, (off, span) in zip(self.master_parameters, self._offsets):
            if not getattr(p, "_pd_acc", False):
                continue
            end = _align(off + span, 64)
            if segs and segs[-1][1] == off:
                segs[-1][1] = end
            else:
                segs.append([off, end])
        return segs

    def step(self, closure=None):
        """One optimizer step on the newest weights (runtime/optimizer.py:122-164)."""
        if self.batch_counter % self.update_interval != self.update_interval - 1:
            self.batch_counter += 1
            return None
        log_timing = self.verbose_freq > 0 and self.batch_counter % self.verbose_freq == 0
        if log_timing:
            start_time = time.time()
        self._collect_foreign_grads()
        grad_scale = 1.0 / self.update_interval
        if self._grad_sync is not None:
            grad_scale *= self._grad_sync(self.grad_arena)
        if self.dtype != torch.float32 and self.loss_scale != 1.0:
            grad_scale /= self.loss_scale
        group = self.base_optimizer.param_groups[0]
        read_slot, write_slot = self.ring.advance()
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        w_dtype = pf.dt(self.arena)
        first = self._steps_taken == 0
        segs = self._segments()
        esz = self.arena.element_size()
        full = len(segs) == 1 and segs[0][0] == 0 and segs[0][1] >= self.numel
        if not full:
            # parameters without a gradient keep their value in the new version
            self.arena[write_slot].copy_(self.arena[read_slot])
        for off, end in segs:
            n = end - off
            arena_p = ctypes.c_void_p(self.arena.data_ptr() + off * esz)
            master_p = ctypes.c_void_p(self.master.data_ptr() + off * 4) if self.master is not None else None
            grad_p = ctypes.c_void_p(self.grad_arena.data_ptr() + off * 4)
            sa_p = ctypes.c_void_p(self.state_a.data_ptr() + off * 4)
            if self.optim_name == "SGD":
                call("pd_opt_sgd_multi_tensor", arena_p, self.slot_stride, read_slot, write_slot, w_dtype, master_p,
                     grad_p, sa_p, n, float(group["lr"]), float(group["momentum"]), float(group["dampening"]),
                     float(group["weight_decay"]), int(bool(group["nesterov"])), int(first), grad_scale, stream)
            else:
                sb_p = ctypes.c_void_p(self.state_b.data_ptr() + off * 4)
                b1, b2 = group["betas"]
                call("pd_opt_adam_multi_tensor", arena_p, self.slot_stride, read_slot, write_slot, w_dtype, master_p,
                     grad_p, sa_p, sb_p, n, float(group["lr"]), float(b1), float(b2), float(group["eps"]),
                     float(group["weight_decay"]), self._steps_taken + 1, grad_scale, stream)
        self._steps_taken += 1
        self.latest_version = self.latest_version.incr()
        self._valid_slots.add(write_slot)
        # The module is left on the newest weights.  Like the reference, step() does not
        # touch current_version (only set_params does, runtime/optimizer.py:108).
        self._point_params(write_slot)
        self.trace.append(("step", self.latest_version.version))
        if log_timing:
            print("Optimizer step took: %.3f" % (time.time() - start_time))
        self.batch_counter += 1
        return None

    # ------------------------------------------------------------------ checkpoints
    def state_dict(self):
        """torch.optim-format state with the momentum / Adam moments read from the arena."""
        sd = self.base_optimizer.state_dict()
        state = {}
        if self._steps_taken > 0:
            for i, (p, (off, _)) in enumerate(zip(self.master_parameters, self._offsets)):
                a = self.state_a.as_strided(p.data.shape, p.data.stride(), off).clone()
                if self.optim_name == "SGD":
                    state[i] = {"momentum_buffer": a}
                else:
                    b = self.state_b.as_strided(p.data.shape, p.data.stride(), off).clone()
                    state[i] = {"step": torch.tensor(float(self._steps_taken)), "exp_avg": a, "exp_avg_sq": b}
        sd["state"] = state
        return sd

    def load_state_dict(self, sd):
        groups = sd["param_groups"]
        for g, saved in zip(self.base_optimizer.param_groups, groups):
            for k, v in saved.items():
                if k != "params":
                    g[k] = v
        state = sd.get("state", {})
        steps = 0
        for i, (p, (off, _)) in enumerate(zip(self.master_parameters, self._offsets)):
            st = state.get(i)
            if not st:
                continue
            a = self.state_a.as_strided(p.data.shape, p.data.stride(), off)
            if self.optim_name == "SGD":
                if st.get("momentum_buffer") is not None:
                    a.copy_(st["momentum_buffer"])
                    steps = max(steps, 1)
            else:
                a.copy_(st["exp_avg"])
                self.state_b.as_strided(p.data.shape, p.data.stride(), off).copy_(st["exp_avg_sq"])
                steps = max(steps, int(st["step"]))
        self._steps_taken = steps

    def resync_from_modules(self):
        """The parameters were overwritten in place (a checkpoint was loaded into the modules after this
        optimizer took them into its arena): make every stashed version, and the fp32 master copy, equal to
        the values the parameters hold now - the state the reference is in when the checkpoint is loaded before
        the optimizer is built (all queue entries are clones of the loaded weights, runtime/optimizer.py:58-62).
        Version numbers and optimizer state are left alone."""
        cur = self._current_slot
        for s in range(self.num_versions):
            if s != cur:
                self.arena[s].copy_(self.arena[cur])
        self._valid_slots = set(range(self.num_versions))
        if self.master is not None:
            for p, (off, _) in zip(self.master_parameters, self._offsets):
                self.master.as_strided(p.data.shape, p.data.stride(), off).copy_(p.data)

    # ------------------------------------------------------------------ full-fidelity checkpoints
    def ring_state_dict(self):
        """Everything a bit-exact resume in the middle of a pipelined epoch needs beyond torch.optim's
        state: every stashed weight version with its number, the fp32 master copy, and the step counters.
        The reference checkpoints between epochs only, where all versions coincide
        (main_with_runtime.py:322-330); this is the in-flight complement."""
        return {
            "num_versions": self.num_versions,
            "latest_version": self.latest_version.version,
            "current_version": self.current_version.version,
            "batch_counter": self.batch_counter,
            "steps_taken": self._steps_taken,
            "arena": self.arena.detach().clone(),
            "master": self.master.detach().clone() if self.master is not None else None,
            "valid_slots": sorted(self._valid_slots),
            "current_slot": self._current_slot,
        }

    def load_ring_state_dict(self, sd):
        if sd["num_versions"] != self.num_versions or sd["arena"].shape != self.arena.shape:
            raise ValueError("version ring of the checkpoint (%d versions, %s) does not match this stage (%d, %s)" % (
                sd["num_versions"], tuple(sd["arena"].shape), self.num_versions, tuple(self.arena.shape)))
        self.arena.copy_(sd["arena"])
        if self.master is not None:
            self.master.copy_(sd["master"])
        self.latest_version = Version(sd["latest_version"])
        self.current_version = Version(sd["current_version"])
        self.batch_counter = sd["batch_counter"]
        self._steps_taken = sd["steps_taken"]
        self.ring = VersionRing(self.num_versions)
        self.ring.latest = self.latest_version.version
        self._valid_slots = set(sd["valid_slots"])
        self._point_params(sd["current_slot"])
