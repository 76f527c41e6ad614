"""``fuse`` and ``decompose``.

``sch.fuse(subgraph, compiler, name)`` turns one matched chain into a single
module.  Compilers:

* ``"native"`` - recognise the chain (bias+GeLU / bias+ReLU, bias + dropout +
  residual add (+ LayerNorm), LayerNorm) and swap in the hand-written
  sm_100a kernel module from :mod:`slapo_b200.ops`; raises if the chain is
  not one of the supported shapes;
* ``"TorchScript"`` - extract the chain and ``torch.jit.script`` it;
* ``None`` - just group the chain in an ``nn.Sequential`` subclass whose class
  name is ``name`` (a structural marker, e.g. for a later ``replace``).

``sch.decompose()`` rewrites an ``nn.Linear`` with bias into "matmul, then an
explicit bias add" sharing the same Parameter objects, so that the add shows
up in the traced graph and can be fused with what follows.

Parity: slapo/primitives/fusion.py:15-98 of the reference (which has the
TorchScript and None compilers only).
"""
from __future__ import annotations

import torch
from torch import nn

from .base import Primitive, register_primitive


_FUNCTION_MODULES = {
    torch.nn.functional.relu: nn.ReLU,
    torch.relu: nn.ReLU,
    torch.nn.functional.gelu: nn.GELU,
    torch.tanh: nn.Tanh,
    torch.nn.functional.silu: nn.SiLU,
    torch.sigmoid: nn.Sigmoid,
}


def _group_as_sequential(sch, chain, gm, name):
    """An ``nn.Sequential`` subclass named ``name``.  A straight chain of module
    calls and single-input activations keeps its members as elements ``0..n-1``;
    anything else is grouped as one extracted graph module.  The first element
    receives every external input of the chain."""

    def forward(self, *args):
        mods = list(self)
        out = mods[0](*args)
        for mod in mods[1:]:
            out = mod(out)
        return out

    seq_cls = type(name, (nn.Sequential,), {"forward": forward})
    members = []
    prev = None
    for path, node in chain:
        owner = sch.mod if not path else sch.get_module(path)
        straight = prev is None or (len(node.all_input_nodes) == 1
                                    and node.all_input_nodes[0] is prev)
        if node.op == "call_module" and straight:
            members.append(owner.get_submodule(node.target))
        elif (node.op == "call_function" and straight and node.target in _FUNCTION_MODULES
              and len(node.args) == 1 and not node.kwargs):
            members.append(_FUNCTION_MODULES[node.target]())
        else:
            return seq_cls(gm)
        prev = node
    return seq_cls(*members)


@register_primitive()
class FusePrimitive(Primitive):
    @staticmethod
    def name():
        return "fuse"

    @staticmethod
    def is_verifiable():
        return True

    @staticmethod
    def apply(sch, subgraph, compiler="TorchScript", name="FusedModule"):
        if not (len(subgraph) == 1 and len(subgraph[0]) > 1):
            raise ValueError("fuse supports vertical fusion only: pass one chain of >1 nodes")
        chain = subgraph[0]
        if compiler == "native":
            from ..ops.fusion_patterns import build_native_module

            new_mod = build_native_module(sch, chain)
        else:
            gm = sch._construct_fx_graph(chain)
            if compiler == "TorchScript":
                new_mod = torch.jit.script(gm)
            elif compiler is None:
                new_mod = _group_as_sequential(sch, chain, gm, name)
            else:
                raise ValueError(f"unknown compiler {compiler}")
        return sch.replace(new_mod, subgraph, name=name)


@register_primitive()
class DecomposePrimitive(Primitive):
    @staticmethod
    def name():
        return "decompose"

    @staticmethod
    def apply(sch):
        from ..ops.linear import LinearWithSeparateBias

        mod = sch.mod
        if not isinstance(mod, nn.Linear):
            raise RuntimeError(f"can only decompose nn.Linear, got {type(mod).__name__}")
        if mod.bias is None or isinstance(mod, LinearWithSeparateBias):
            return
        new_mod = LinearWithSeparateBias(mod.in_features, mod.out_features, device="meta")
        new_mod.weight, new_mod.bias = mod.weight, mod.bias
        sch.replace(new_mod)
