"""``shard``, ``sync`` and ``fork_rng``: the tensor-parallel primitives.

Parity: slapo/primitives/tensor_parallel.py:14-194 of the reference.
"""
from __future__ import annotations

import functools


from ..parallel.shard_methods import (apply_shard_method, apply_sync_method,
                                      new_or_get_tied_param)
from ..random import get_cuda_rng_tracker
from ..utils.common import transfor_param_tags
from .base import Primitive, register_primitive


@register_primitive()
class ShardPrimitive(Primitive):
    """``sch.shard(tensor_name, axis)`` keeps this rank's 1/world_size slice
    of a parameter or buffer along ``axis``.

    The slice is ``tensor.chunk(world_size, axis)[rank]``; the new parameter
    remembers ``orig_shape`` so that checkpoints can be consolidated and
    delayed initialisation can create the full tensor, slice it and stay
    consistent with an unsharded run."""

    @staticmethod
    def name():
        return "shard"

    @staticmethod
    def is_verifiable():
        return True

    @staticmethod
    def init_metadata():
        return {}

    @staticmethod
    def apply(sch, tensor_name: str, axis: int):
        mod = sch.mod
        is_param = tensor_name in mod._parameters
        if not is_param and tensor_name not in mod._buffers:
            raise KeyError(f"{sch.path or '<root>'} has no parameter or buffer '{tensor_name}'")
        tensor = getattr(mod, tensor_name)
        if tensor is None:
            raise ValueError(f"'{tensor_name}' of {sch.path} is None")
        axis = axis if axis >= 0 else axis + tensor.dim()
        size = tensor.shape[axis]
        if size % sch.world_size != 0:
            raise ValueError(
                f"axis {axis} of {sch.path}.{tensor_name} has size {size}, "
                f"not divisible by the group size {sch.world_size}")
        sharded_size = size // sch.world_size
        apply_shard_method("preproc", sch, tensor_name, sharded_size, axis)
        piece = tensor.detach().narrow(axis, sch.rank * sharded_size, sharded_size).contiguous()
        orig_shape = getattr(tensor, "orig_shape", tuple(tensor.shape))
        if is_param:
            new_param = new_or_get_tied_param(sch, tensor, piece)
            transfor_param_tags(sch, tensor, new_param)
            mod.register_parameter(tensor_name, new_param)
            sch.annotate(tensor_name, "orig_shape", tuple(orig_shape))
        else:
            persistent = tensor_name not in mod._non_persistent_buffers_set
            mod.register_buffer(tensor_name, piece, persistent=persistent)
            piece.orig_shape = tuple(orig_shape)
        meta = sch.metadata.primitives["shard"]
        if meta.get(tensor_name, axis) != axis:
            raise RuntimeError(
                f"{sch.path}.{tensor_name} is already sharded along axis {meta[tensor_name]}")
        meta[tensor_name] = axis
        apply_shard_method("postproc", sch, tensor_name, sharded_size, axis)
        apply_shard_method("infer_and_set_output_type", sch, tensor_name, sharded_size, axis)


@register_primitive()
class SyncPrimitive(Primitive):
    """``sch.sync(mode, sync_op_or_fn, **kwargs)`` places a collective (or a
    user hook) before the forward (``fwd_pre``), after it (``fwd_post``) or
    on the input gradient (``bwd_post``).

    String ops: ``all_gather`` (axis, tensor_parallel_output_grad),
    ``reduce_scatter`` (axis), ``scatter`` (axis), ``all_reduce`` and the
    reshards ``"RS->SR"`` etc.  ``axis`` counts dimensions of the tensor the
    collective acts on."""

    @staticmethod
    def name():
        return "sync"

    @staticmethod
    def init_metadata():
        return []

    @staticmethod
    def apply(sch, mode, sync_op_or_fn, **kwargs):
        if mode not in ("fwd_pre", "fwd_post", "bwd_post"):
            raise ValueError(f"unsupported sync mode '{mode}'")
        record = sch.metadata.primitives.get("sync")
        if record is None:
            record = sch.metadata.primitives["sync"] = []
        apply_sync_method(sch, mode, sync_op_or_fn, **kwargs)
        record.append((mode, sync_op_or_fn if isinstance(sync_op_or_fn, str) else "custom",
                       dict(kwargs)))


@register_primitive()
class ForkRNGPrimitive(Primitive):
    """``sch.fork_rng()`` runs the module's forward under the tensor-parallel
    RNG stream, so dropout masks differ between TP ranks (needed when the
    activation itself is sharded)."""

    @staticmethod
    def name():
        return "fork_rng"

    @staticmethod
    def apply(sch):
        mod = sch.mod
        if getattr(mod, "_slapo_rng_forked", False):
            return
        inner = mod.forward

        @functools.wraps(inner)
        def forked_forward(*args, **kwargs):
            with get_cuda_rng_tracker().fork():
                return inner(*args, **kwargs)

        mod.forward = forked_forward
        mod._slapo_rng_forked = True
        mod.traceable = False
