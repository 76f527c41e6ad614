"""``checkpoint``: activation checkpointing of a module or a matched sub-graph.

Parity: slapo/primitives/checkpoint.py:12-58 of the reference.
"""
from __future__ import annotations

import functools
import inspect

import torch
from torch import nn
from torch.utils._pytree import tree_flatten

from ..checkpoint import checkpoint as checkpoint_fn
from .base import Primitive, register_primitive


class CheckPointWrapper(nn.Module):
    """Runs the wrapped module under activation checkpointing.

    Keyword arguments are bound to the wrapped forward's signature and passed
    positionally (checkpointing with RNG replay is positional); a custom
    ``order_args_fn(*args, **kwargs) -> list`` overrides the binding.  What lands in
    a catch-all ``**kwargs`` of the wrapped forward (Hugging Face layers take flags and
    position tensors that way) is handed on by name outside the checkpointed argument
    list - allowed as long as none of it requires a gradient."""

    traceable = False

    def __init__(self, mod: nn.Module, order_args_fn=None):
        super().__init__()
        self.mod = mod
        self.order_args_fn = order_args_fn
        try:
            self._sig = inspect.signature(mod.forward)
        except (TypeError, ValueError):
            self._sig = None

    def _ordered(self, args, kwargs):
        """``(positional argument list, extra keyword arguments)``."""
        if self.order_args_fn is not None:
            return list(self.order_args_fn(*args, **kwargs)), {}
        if not kwargs:
            return list(args), {}
        if self._sig is None:
            raise ValueError("cannot order keyword arguments; pass order_args_fn")
        bound = self._sig.bind(*args, **kwargs)
        bound.apply_defaults()
        ordered, extras = [], {}
        for name, par in self._sig.parameters.items():
            if par.kind is par.VAR_POSITIONAL:
                ordered += list(bound.arguments.get(name, ()))
            elif par.kind is par.VAR_KEYWORD:
                extras = dict(bound.arguments.get(name) or {})
                if any(torch.is_tensor(t) and t.requires_grad
                       for t in tree_flatten(extras)[0]):
                    raise ValueError(
                        f"keyword arguments {sorted(extras)} fall into **{name} of the "
                        "checkpointed forward and carry gradients: they cannot be "
                        "checkpointed positionally; pass order_args_fn")
            elif par.kind is par.KEYWORD_ONLY:
                extras[name] = bound.arguments[name]
            else:
                ordered.append(bound.arguments[name])
        return ordered, extras

    def forward(self, *args, **kwargs):
        ordered, extras = self._ordered(args, kwargs)
        for value in list(ordered) + list(extras.values()):
            if hasattr(value, "get_seq_length") and hasattr(value, "update"):
                raise ValueError(
                    f"a key / value cache ({type(value).__name__}) is passed into a checkpointed "
                    "layer: the layer runs twice and would append to it twice; switch the "
                    "model's use_cache off for training")
        if extras:
            return checkpoint_fn(functools.partial(self.mod, **extras), *ordered)
        return checkpoint_fn(self.mod, *ordered)


@register_primitive()
class CheckpointPrimitive(Primitive):
    """``sch.checkpoint()`` wraps this module; ``sch.checkpoint(subgraph)``
    extracts the matched chain into its own module first and wraps that."""

    @staticmethod
    def name():
        return "checkpoint"

    @staticmethod
    def apply(sch, subgraph=None, order_args_fn=None):
        if subgraph is None:
            if isinstance(sch.mod, CheckPointWrapper):
                return
            sch.replace(CheckPointWrapper(sch.mod, order_args_fn))
            return
        if len(subgraph) != 1:
            raise ValueError("checkpoint takes exactly one matched sub-graph")
        chain = subgraph[0] if isinstance(subgraph[0], list) else subgraph
        gm = sch._construct_fx_graph(chain)
        sch.replace(CheckPointWrapper(gm, order_args_fn), [chain], name="CheckPointWrapper")
