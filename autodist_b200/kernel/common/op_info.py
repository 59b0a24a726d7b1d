"""Which optimizers the runtime recognises and how their state is laid out.

The reference keys on TensorFlow update-op types (``autodist/kernel/common/op_info.py:24-117``);
here the key is the ``torch.optim`` class. ``FUSED`` optimizers have a hand-written
sm_100a update kernel (dense and row-sparse forms); the others run as per-shard
``torch.optim`` instances re-created from the captured constructor arguments.
"""
import torch

# optimizer class name -> names of per-parameter state tensors shaped like the parameter
SLOT_NAMES = {
    "SGD": ("momentum_buffer",),
    "Adam": ("exp_avg", "exp_avg_sq", "max_exp_avg_sq"),
    "AdamW": ("exp_avg", "exp_avg_sq", "max_exp_avg_sq"),
    "Adagrad": ("sum",),
    "RMSprop": ("square_avg", "momentum_buffer", "grad_avg"),
    "Adadelta": ("square_avg", "acc_delta"),
    "Adamax": ("exp_avg", "exp_inf"),
    "NAdam": ("exp_avg", "exp_avg_sq"),
    "RAdam": ("exp_avg", "exp_avg_sq"),
    "ASGD": ("ax",),
    "Rprop": ("prev", "step_size"),
    "SparseAdam": ("exp_avg", "exp_avg_sq"),
    "LBFGS": (),
}

FUSED = ("SGD", "Adam", "AdamW", "Adagrad")

DENSE_UPDATE_OPTIMIZERS = tuple(n for n in SLOT_NAMES if n not in ("SparseAdam", "LBFGS"))
# Optimizers whose update of untouched rows is the identity, so a row-sparse gradient may be
# applied to the touched rows only (the reference's ResourceSparseApply* family).
SPARSE_UPDATE_OPTIMIZERS = ("SGD", "Adagrad", "SparseAdam")

CONTROL_FLOW_TARGETS = (torch.cond,) if hasattr(torch, "cond") else ()


def slot_names(optimizer_cls):
    return SLOT_NAMES.get(optimizer_cls.__name__, ())


def supports_sparse_rows(optimizer):
    name = type(optimizer).__name__
    if name == "SGD":
        g = optimizer.param_groups[0]
        return g.get("momentum", 0) == 0 and g.get("weight_decay", 0) == 0
    return name in SPARSE_UPDATE_OPTIMIZERS
