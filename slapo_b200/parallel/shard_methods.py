"""Per-module-class rules for ``shard`` and ``sync``.

``shard`` only slices a tensor; what that *means* for the module (new
``out_features``, whether its output is now a partition along some axis or a
partial sum) depends on the module class and is described by a
``ShardMethod`` registered with ``@register_shard_method(cls)``.  The inferred
output kind lets ``sync`` reject collectives that cannot be right, e.g. an
all-reduce on a partitioned output.

``sync`` with a string op attaches a ``SyncHook`` (a callable object that
records mode / op / arguments) as a forward(-pre) hook, so that the schedule
can be printed, verified and later *lowered*: on a B200 the pair
"sharded Linear + adjacent collective" is rewritten into one fused
GEMM+collective kernel by :mod:`slapo_b200.parallel.lowering`.

Parity: slapo/sharding/shard_ops.py:26-649 of the reference.
"""
from __future__ import annotations

import copy
from functools import partial

import torch
import torch.distributed as dist
from torch import nn

from ..logger import get_logger
from .reshard_ops import parse_reshard
from .sync_ops import (all_gather_forward_output, reduce_backward_grad,
                       reduce_forward_output, reduce_scatter_forward_output,
                       scatter_forward_output)

logger = get_logger("sharding")

SHARD_METHODS: dict[type, type] = {}


def register_shard_method(module_cls, override: bool = False):
    def decorator(method_cls):
        if module_cls is None:  # optional class that is not importable
            return method_cls
        if not issubclass(method_cls, ShardMethod):
            raise ValueError(f"{method_cls} must subclass ShardMethod")
        if module_cls in SHARD_METHODS and not override:
            raise ValueError(f"shard method of {module_cls} already registered")
        SHARD_METHODS[module_cls] = method_cls
        return method_cls

    return decorator


def dispatch_shard_method_cls(sch):
    best, best_depth = ShardMethod, -1
    for cls, method in SHARD_METHODS.items():
        if isinstance(sch.mod, cls):
            depth = len(cls.__mro__)
            if depth > best_depth:  # most derived registered class wins
                best, best_depth = method, depth
    return best


def apply_shard_method(method_name, sch, *args, **kwargs):
    return getattr(dispatch_shard_method_cls(sch), method_name)(sch, *args, **kwargs)


def apply_sync_method(sch, mode, sync_op_or_fn, **kwargs):
    return dispatch_shard_method_cls(sch).sync(sch, mode, sync_op_or_fn, **kwargs)


# ---------------------------------------------------------------------- #
class SyncFn:
    """``tensor -> tensor`` collective bound to a group.  Deep copies share
    the process group (groups cannot be copied)."""

    def __init__(self, func, op, group, **kwargs):
        self.func, self.sync_op, self.group, self.sync_kwargs = func, op, group, kwargs

    def __call__(self, tensor):
        return self.func(tensor)

    def __deepcopy__(self, memo):
        return self

    def __repr__(self):
        kw = ", ".join(f"{k}={v}" for k, v in self.sync_kwargs.items())
        return f"{self.sync_op}({kw})"


class SyncHook:
    """A forward(-pre) hook that applies one collective and remembers which."""

    def __init__(self, mode, op, fn, group, **kwargs):
        self.mode, self.op, self.fn, self.group, self.kwargs = mode, op, fn, group, kwargs

    def __deepcopy__(self, memo):
        return self

    def __call__(self, module, inputs, output=None):
        if self.mode == "fwd_post":
            return self._on_first_tensor(output)
        first = self.fn(inputs[0])
        return (first,) + tuple(inputs[1:])

    def meta_shape(self, shape):
        """The shape this hook turns ``shape`` into (the module's first input for a forward-pre
        hook, its main output for a forward hook): what a shape-propagating tracer needs to
        know about a collective that it cannot run on meta tensors."""
        axis = self.kwargs.get("axis", 0)
        if self.op not in ("all_gather", "scatter", "reduce_scatter") or len(shape) <= axis:
            return tuple(shape)
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        out = list(shape)
        out[axis] = out[axis] * world if self.op == "all_gather" else out[axis] // world
        return tuple(out)

    def _on_first_tensor(self, output):
        """The collective applies to the module's main output: the tensor itself, the first
        element of a tuple (a Hugging Face layer returns ``(hidden_states, ...)``) or the first
        tensor entry of a dict-like output (``last_hidden_state`` of a ``ModelOutput``)."""
        if isinstance(output, (tuple, list)) and output and torch.is_tensor(output[0]):
            return type(output)([self.fn(output[0]), *output[1:]])
        if hasattr(output, "keys") and not torch.is_tensor(output):
            for key in output.keys():
                if torch.is_tensor(output[key]):
                    new = copy.copy(output)
                    new[key] = self.fn(output[key])
                    return new
        return self.fn(output)

    def __repr__(self):
        extra = ", ".join(f"{k}={v}" for k, v in self.kwargs.items())
        return f"SyncHook({self.mode}, {self.op}{', ' + extra if extra else ''})"


def _shard_meta(sch):
    meta = sch.metadata.primitives.get("shard")
    if meta is None:
        meta = sch.metadata.primitives["shard"] = {}
    return meta


def validate_sync(sch, mode, op, axis=None):
    """Reject collectives that contradict the inferred output kind."""
    meta = _shard_meta(sch)
    kind = meta.get("output_type")
    if mode == "fwd_post" and op == "scatter" and kind is not None:
        raise ValueError(f"output of {sch.path} cannot be scattered: its parameters are sharded")
    if kind is None:
        return
    if mode == "fwd_post" and op == "all_gather":
        if kind != "partition":
            raise ValueError(f"output of {sch.path} is a partial sum; it cannot be all-gathered")
        want = meta.get("gather_axis")
        if want != axis and not (want == -1 and axis is not None and axis >= 1):
            raise ValueError(
                f"output of {sch.path} has to be gathered along axis "
                f"{want}, but {axis} is requested")
    elif mode == "fwd_post" and op == "reduce_scatter" and kind == "partition":
        raise ValueError(f"output of {sch.path} is a partition; it cannot be reduce-scattered")
    elif mode == "fwd_pre" and op == "all_gather" and kind == "partial":
        raise ValueError(
            f"{sch.path} is sharded along its input dimension and expects a partitioned "
            "input; all-gathering the input is wrong")
    elif mode == "fwd_post" and op == "all_reduce" and kind == "partition":
        raise ValueError(f"output of {sch.path} is a partition; it cannot be all-reduced")


def make_sync_fn(sch, mode, op, **kwargs):
    """(effective hook mode, ``SyncFn``) for a string op."""
    eff_mode, func = _make_sync_callable(sch, mode, op, **kwargs)
    return eff_mode, SyncFn(func, op, sch.group, **kwargs)


def _make_sync_callable(sch, mode, op, **kwargs):
    group = sch.group
    axis = kwargs.get("axis", 0)
    if mode in ("fwd_post", "fwd_pre"):
        if op == "all_gather":
            validate_sync(sch, mode, op, axis)
            return mode, partial(
                all_gather_forward_output, dim=axis, group=group,
                tensor_parallel_output_grad=kwargs.get("tensor_parallel_output_grad", True))
        if "->" in op:
            return mode, parse_reshard(op, group)
        if op == "scatter" and mode == "fwd_pre":
            # keep this rank's part of the first input (the start of a sequence-parallel
            # region in front of a block); the gradient is gathered again
            return mode, partial(scatter_forward_output, dim=axis, group=group)
        if mode == "fwd_post":
            if op == "reduce_scatter":
                validate_sync(sch, mode, op)
                return mode, partial(reduce_scatter_forward_output, dim=axis, group=group)
            if op == "scatter":
                validate_sync(sch, mode, op)
                return mode, partial(scatter_forward_output, dim=axis, group=group)
            if op == "all_reduce":
                validate_sync(sch, mode, op)
                return mode, partial(reduce_forward_output, group=group)
    elif mode == "bwd_post":
        if op == "all_reduce":
            # an identity whose gradient is all-reduced, applied to the input:
            # clearer semantics than a module backward hook
            validate_sync(sch, mode, op)
            return "fwd_pre", partial(reduce_backward_grad, group=group)
    raise ValueError(f"invalid sync op '{op}' for mode '{mode}' at {sch.path}")


class ShardMethod:
    """Default rules: no attribute fix-up, output kind unknown."""

    @staticmethod
    def preproc(sch, param_name, sharded_size, axis):
        return None

    @staticmethod
    def postproc(sch, param_name, sharded_size, axis):
        return None

    @staticmethod
    def infer_output_type(sch, param_name, sharded_size, axis):
        return None, None

    @staticmethod
    def infer_and_set_output_type(sch, param_name, sharded_size, axis):
        kind, gather_axis = apply_shard_method(
            "infer_output_type", sch, param_name, sharded_size, axis)
        meta = _shard_meta(sch)
        if kind is not None:
            if meta.get("output_type", kind) != kind:
                raise RuntimeError(
                    f"output of {sch.path} is already '{meta['output_type']}', "
                    f"sharding {param_name} along {axis} would make it '{kind}'")
            meta["output_type"] = kind
        if gather_axis is not None:
            if kind != "partition":
                raise RuntimeError("a gather axis only makes sense for a partitioned output")
            if meta.get("gather_axis", gather_axis) != gather_axis:
                raise RuntimeError(
                    f"output of {sch.path} has to be gathered along axis "
                    f"{meta['gather_axis']}, not {gather_axis}")
            meta["gather_axis"] = gather_axis

    @staticmethod
    def sync(sch, mode, sync_op_or_fn, **kwargs):
        if isinstance(sync_op_or_fn, str):
            eff_mode, fn = make_sync_fn(sch, mode, sync_op_or_fn, **kwargs)
            hook = SyncHook(eff_mode, sync_op_or_fn if mode != "bwd_post" else "bwd_all_reduce",
                            fn, sch.group, **kwargs)
            mode = eff_mode
        else:
            hook = sync_op_or_fn
        if mode == "fwd_pre":
            sch.mod.register_forward_pre_hook(hook)
        elif mode == "fwd_post":
            sch.mod.register_forward_hook(hook)
        elif mode == "bwd_post":
            sch.mod.register_full_backward_hook(hook)
        else:
            raise ValueError(f"unsupported sync mode {mode}")


# ---------------------------------------------------------------------- #
def _sync_with_deferred_bias(sch, mode, sync_op_or_fn, make_replacement, **kwargs):
    """Row-parallel layers produce partial sums; a bias must be added *after*
    the reduction or it would be counted world_size times.  So a fwd_post
    collective on such a layer swaps the layer for a variant that computes
    matmul -> collective -> + bias."""
    mod = sch.mod
    partial_out = _shard_meta(sch).get("output_type") == "partial"
    if mode != "fwd_post" or not partial_out or getattr(mod, "bias", None) is None:
        return ShardMethod.sync(sch, mode, sync_op_or_fn, **kwargs)
    if not isinstance(sync_op_or_fn, str):
        raise ValueError(
            f"{sch.path} has a bias and a partial-sum output: only string sync ops can "
            "be ordered before the bias add")
    _, fn = make_sync_fn(sch, mode, sync_op_or_fn, **kwargs)
    if hasattr(mod, "sync_fn"):  # already a matmul->sync->bias layer
        mod.sync_fn = fn
        return None
    new_mod = make_replacement(mod, fn)
    sch.replace(new_mod)
    return None


@register_shard_method(nn.Linear)
class ShardLinear(ShardMethod):
    @staticmethod
    def postproc(sch, param_name, sharded_size, axis):
        if param_name == "weight":
            if axis == 0:
                sch.mod.out_features = sharded_size
            else:
                sch.mod.in_features = sharded_size
        elif param_name == "bias":
            sch.mod.out_features = sharded_size

    @staticmethod
    def infer_output_type(sch, param_name, sharded_size, axis):
        if param_name == "bias":
            return "partition", -1
        return ("partition", -1) if axis == 0 else ("partial", None)

    @staticmethod
    def sync(sch, mode, sync_op_or_fn, **kwargs):
        from ..ops.linear import LinearWithSyncFunc

        def make(mod, fn):
            new = LinearWithSyncFunc(mod.in_features, mod.out_features, bias=True,
                                     device="meta", sync_fn=fn)
            new.weight, new.bias = mod.weight, mod.bias
            return new

        return _sync_with_deferred_bias(sch, mode, sync_op_or_fn, make, **kwargs)


@register_shard_method(nn.Conv2d)
class ShardConv2d(ShardMethod):
    @staticmethod
    def postproc(sch, param_name, sharded_size, axis):
        mod = sch.mod
        if param_name == "bias":
            mod.out_channels = sharded_size
            return
        out_axis = 1 if getattr(mod, "transposed", False) else 0
        if axis == out_axis:
            mod.out_channels = sharded_size
        else:
            mod.in_channels = sharded_size

    @staticmethod
    def infer_output_type(sch, param_name, sharded_size, axis):
        out_axis = 1 if getattr(sch.mod, "transposed", False) else 0
        if param_name == "bias" or axis == out_axis:
            return "partition", 1
        return "partial", None


@register_shard_method(nn.BatchNorm2d)
class ShardBatchNorm2d(ShardMethod):
    @staticmethod
    def preproc(sch, param_name, sharded_size, axis):
        if axis != 0:
            raise ValueError("BatchNorm2d tensors are one-dimensional: shard axis must be 0")

    @staticmethod
    def postproc(sch, param_name, sharded_size, axis):
        sch.mod.num_features = sharded_size

    @staticmethod
    def infer_output_type(sch, param_name, sharded_size, axis):
        return "partition", 1


@register_shard_method(nn.Embedding)
class ShardEmbedding(ShardMethod):
    """axis 0 = vocabulary-parallel (each rank owns a range of ids and
    contributes zeros elsewhere: partial sum); axis 1 = hidden-parallel."""

    @staticmethod
    def postproc(sch, param_name, sharded_size, axis):
        mod = sch.mod
        if axis == 0:
            mod.num_embeddings = sharded_size
            mod.vocab_start_index = sch.rank * sharded_size
            mod.vocab_end_index = (sch.rank + 1) * sharded_size
            if mod.padding_idx is not None:
                lo = mod.vocab_start_index
                mod.padding_idx = mod.padding_idx - lo if lo <= mod.padding_idx < lo + sharded_size else None
        else:
            mod.embedding_dim = sharded_size

    @staticmethod
    def infer_output_type(sch, param_name, sharded_size, axis):
        return ("partial", None) if axis == 0 else ("partition", -1)


def _conv1d_cls():
    try:
        from ..models.gpt import Conv1D

        return Conv1D
    except Exception:  # pragma: no cover
        return None


@register_shard_method(_conv1d_cls())
class ShardConv1D(ShardMethod):
    """GPT-2 ``Conv1D``: the weight is ``[in, out]``, so axis 1 splits the
    output features (partitioned output) and axis 0 the input features
    (partial sums)."""

    @staticmethod
    def postproc(sch, param_name, sharded_size, axis):
        if param_name == "bias" or axis == 1:
            sch.mod.nf = sharded_size
        else:
            sch.mod.nx = sharded_size

    @staticmethod
    def infer_output_type(sch, param_name, sharded_size, axis):
        if param_name == "bias" or axis == 1:
            return "partition", -1
        return "partial", None

    @staticmethod
    def sync(sch, mode, sync_op_or_fn, **kwargs):
        from ..ops.linear import Conv1DWithSyncFunc

        def make(mod, fn):
            new = Conv1DWithSyncFunc(mod.nf, mod.nx, device="meta", sync_fn=fn)
            new.weight, new.bias = mod.weight, mod.bias
            return new

        return _sync_with_deferred_bias(sch, mode, sync_op_or_fn, make, **kwargs)


@register_shard_method(nn.LayerNorm)
class ShardLayerNorm(ShardMethod):
    @staticmethod
    def preproc(sch, param_name, sharded_size, axis):
        raise ValueError("LayerNorm normalises over the hidden dimension and cannot be sharded")


# ---------------------------------------------------------------------- #
def new_or_get_tied_param(sch, old_param, new_tensor):
    """Parameter to register in place of ``old_param`` after slicing.

    If ``old_param`` is shared by several modules, the first shard creates the
    replacement and later shards of the other aliases get the same object, so
    tied weights stay tied.  A differing slice shape means the aliases were
    sharded inconsistently."""
    tie = sch.metadata.tie_weights
    if old_param in tie:
        current = tie[old_param]
        if current is not old_param:
            if tuple(current.shape) != tuple(new_tensor.shape):
                raise RuntimeError(
                    f"tied parameter sharded inconsistently: {tuple(current.shape)} vs "
                    f"{tuple(new_tensor.shape)} at {sch.path}")
            return current
        new_param = nn.Parameter(new_tensor, requires_grad=old_param.requires_grad)
        tie[old_param] = new_param
        return new_param
    return nn.Parameter(new_tensor, requires_grad=old_param.requires_grad)
