"""The two optimizer front ends the driver scripts construct (runtime/sgd.py:8-24, runtime/adam.py:8-22).

Each only names its hyper-parameters and hands them to OptimizerWithWeightStashing, which keeps a
torch.optim object for `param_groups` / checkpoints and runs the fused ring kernel for the update."""
from torch.optim.optimizer import required

from .optimizer import OptimizerWithWeightStashing


def _front_end(optim_name, self, common, hyper, update_interval=None):
    modules, master_parameters, model_parameters, loss_scale, num_versions, verbose_freq, macrobatch = common
    OptimizerWithWeightStashing.__init__(self, optim_name, modules, master_parameters, model_parameters,
                                         loss_scale, num_versions, verbose_freq, macrobatch,
                                         update_interval=update_interval, **hyper)


class SGDWithWeightStashing(OptimizerWithWeightStashing):
    """SGD (momentum, dampening, L2 weight decay, optional Nesterov) with weight stashing."""

    def __init__(self, modules, master_parameters, model_parameters, loss_scale, num_versions,
                 lr=required, momentum=0, dampening=0, weight_decay=0, nesterov=False,
                 verbose_freq=0, macrobatch=False, update_interval=None):
        _front_end("SGD", self,
                   (modules, master_parameters, model_parameters, loss_scale, num_versions, verbose_freq, macrobatch),
                   dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay, nesterov=nesterov),
                   update_interval)


class AdamWithWeightStashing(OptimizerWithWeightStashing):
    """Adam (L2 weight decay, eps 1e-8) with weight stashing."""

    def __init__(self, modules, master_parameters, model_parameters, loss_scale, num_versions,
                 lr=required, betas=(0.9, 0.999), weight_decay=0, verbose_freq=0, macrobatch=False,
                 update_interval=None):
        _front_end("Adam", self,
                   (modules, master_parameters, model_parameters, loss_scale, num_versions, verbose_freq, macrobatch),
                   dict(lr=lr, betas=betas, weight_decay=weight_decay), update_interval)
