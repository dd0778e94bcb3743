"""The 1F1B training loop a driver script runs around StageRuntime.

`train_1f1b` restates the loop of the reference's
runtime/image_classification/main_with_runtime.py:359-421 (warm-up forwards,
steady state of forward / load_old / backward / load_new / step, drain) so that
tests and benchmarks can drive a stage without the driver script.
`LocalPipeline` runs every stage of a pipeline inside one process on one GPU
(transport "local"), interleaving the per-stage programs in dependency order;
it produces the same numbers as one process per stage because each stage's own
operation order is unchanged.
"""

from . import communication


def stage_program(num_warmup, n):
    """Per-stage operation list for n minibatches: ('F', i) / ('B', i)."""
    prog = [("F", i) for i in range(num_warmup)]
    for i in range(n - num_warmup):
        prog.append(("F", num_warmup + i))
        prog.append(("B", i))
    for i in range(num_warmup):
        prog.append(("B", n - num_warmup + i))
    return prog


def backward_step(r, optimizer):
    """One backward pass with weight stashing (main_with_runtime.py:406-413)."""
    optimizer.zero_grad()
    optimizer.load_old_params()
    r.run_backward()
    optimizer.load_new_params()
    optimizer.step()


def train_1f1b(r, optimizer, n, on_forward=None, no_input_pipelining=False):
    """Runs n minibatches on one stage.  on_forward(i, r) is called after each steady-state forward."""
    w = 0 if no_input_pipelining else r.num_warmup_minibatches
    for _ in range(w):
        r.run_forward()
    for i in range(n - w):
        r.run_forward()
        if on_forward is not None:
            on_forward(i, r)
        backward_step(r, optimizer)
    for _ in range(w):
        backward_step(r, optimizer)
    r.wait()


class LocalPipeline:
    """All stages of a pipeline in one process: list of (StageRuntime, optimizer) in rank order."""

    def __init__(self, workers):
        self.workers = workers

    def run(self, n_per_rank, on_loss=None):
        """n_per_rank[rank] minibatches on each rank (see StageRuntime.num_iterations)."""
        programs = [stage_program(r.num_warmup_minibatches, n_per_rank[k]) for k, (r, _) in enumerate(self.workers)]
        pcs = [0] * len(self.workers)
        for k, (r, _) in enumerate(self.workers):
            r.train(n_per_rank[k])
        progress = True
        while progress:
            progress = False
            for k, (r, opt) in enumerate(self.workers):
                while pcs[k] < len(programs[k]):
                    kind, i = programs[k][pcs[k]]
                    if kind == "F":
                        if r.comm_handler is not None and r.stage > 0 and not r.comm_handler.forward_ready():
                            break
                        r.run_forward()
                        if r.is_criterion and on_loss is not None:
                            on_loss(k, i, r)
                    else:
                        if r.comm_handler is not None and r.stage < r.num_stages - 1 \
                                and not r.comm_handler.backward_ready(r.backward_minibatch_id):
                            break
                        backward_step(r, opt)
                    pcs[k] += 1
                    progress = True
        stuck = [k for k in range(len(pcs)) if pcs[k] < len(programs[k])]
        if stuck:
            raise RuntimeError("pipeline deadlocked; ranks %s did not finish" % stuck)


def reset_local():
    communication.reset_local_fabric()
