"""Pattern language for ``Schedule.find``.

* ``Pattern`` – subclass it like an ``nn.Module``; its ``forward`` describes
  the dataflow to look for and its sub-modules match modules of the same type.
* ``ModulePattern(regex)`` – a sub-module placeholder that matches any
  ``call_module`` node whose target matches ``regex``.
* ``call_module(regex, *args)`` – the same inside a plain pattern function.

Parity: slapo/pattern.py:7-22 of the reference.
"""
from __future__ import annotations

import torch.fx
from torch import nn


class Pattern(nn.Module):
    def forward(self, *args):  # pragma: no cover - interface
        raise NotImplementedError


class ModulePattern(Pattern):
    def __init__(self, name: str):
        super().__init__()
        self.name = name
        # never traced into
        self.traceable = False

    def forward(self, *args):
        return args[0] if args else None


def call_module(mod_name: str, *args):
    """Placeholder for "a call of a sub-module whose name matches mod_name".

    Under symbolic tracing (any argument is an ``fx.Proxy``) the call records
    itself as a ``call_function`` node, so pattern functions need no
    ``torch.fx.wrap`` registration in the caller's module.
    """
    for arg in args:
        if isinstance(arg, torch.fx.Proxy):
            return arg.tracer.create_proxy(
                "call_function", call_module, (mod_name,) + tuple(args), {}
            )
    raise RuntimeError("call_module is only meaningful inside a pattern function")
