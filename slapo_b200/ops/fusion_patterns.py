"""Recognisers behind ``sch.fuse(subgraph, compiler="native")``.

A matched chain is copied into a stand-alone graph and classified by the
sequence of operations it contains; a supported sequence is swapped for a
module that calls the hand-written sm_100a kernel of
:mod:`slapo_b200.ops.functional`:

==============================================  ==============================
chain                                           kernel
==============================================  ==============================
``x + bias`` -> GeLU (erf / tanh) or ReLU       ``bias_act``
``[x + bias ->] dropout -> + residual``         ``bias_dropout_add``
``[x + bias ->] dropout -> + residual -> LN``   ``dropout_add_layer_norm``
==============================================  ==============================

Anything else raises ``NotImplementedError`` naming the sequence that was
seen, so that a recipe never silently falls back to an unfused path.  The
reference offers TorchScript/nvFuser for these chains
(slapo/primitives/fusion.py:15-75, slapo/op/bias_gelu.py:1-60 of the reference).
"""
from __future__ import annotations

import operator

import torch
import torch.nn.functional as F
from torch import fx, nn

from . import functional as NF

_ADD_FUNCS = (operator.add, torch.add, operator.iadd)


def _classify(gm: fx.GraphModule, node: fx.Node):
    """``(kind, attrs)`` of one node of the extracted chain."""
    if node.op == "call_function":
        if node.target in _ADD_FUNCS:
            return "add", {}
        if node.target is F.gelu:
            approx = node.kwargs.get("approximate", node.args[1] if len(node.args) > 1 else "none")
            return "act", {"act": "gelu" if approx == "none" else "gelu_new"}
        if node.target in (F.relu, torch.relu):
            return "act", {"act": "relu"}
        if node.target is F.dropout:
            p = node.kwargs.get("p", node.args[1] if len(node.args) > 1 else 0.5)
            training = node.kwargs.get("training", node.args[2] if len(node.args) > 2 else True)
            return "dropout", {"p": float(p), "training": training}
        if node.target is F.layer_norm:
            return "layer_norm", {"functional": True}
    elif node.op == "call_method" and node.target in ("add", "add_"):
        return "add", {}
    elif node.op == "call_module":
        mod = gm.get_submodule(node.target)
        if isinstance(mod, nn.GELU):
            return "act", {"act": "gelu" if mod.approximate == "none" else "gelu_new"}
        if isinstance(mod, nn.ReLU):
            return "act", {"act": "relu"}
        if isinstance(mod, nn.Dropout):
            return "dropout", {"p": float(mod.p), "training": None, "module": mod}
        if isinstance(mod, nn.LayerNorm):
            return "layer_norm", {"module": mod}
    return f"{node.op}:{getattr(node.target, '__name__', node.target)}", {}


def _split_bias(a, b):
    """Of the two operands of ``x + bias`` the bias is the one-dimensional one."""
    return (a, b) if b.dim() == 1 else (b, a)


class NativeBiasAct(nn.Module):
    """``act(x + bias)`` through the fused kernel (backward computes dx and the
    bias gradient in one pass)."""

    def __init__(self, act):
        super().__init__()
        self.act = act

    def forward(self, a, b):
        x, bias = _split_bias(a, b)
        return NF.bias_act(x, bias, self.act)

    def extra_repr(self):
        return f"act={self.act}"


class NativeBiasDropoutAdd(nn.Module):
    """``dropout(x [+ bias]) + residual`` with optional trailing LayerNorm.

    ``order`` lists, for each external input of the chain in the order the
    chain reads them, which role it plays (``"x"``, ``"bias"``, ``"residual"``;
    ``"x|bias"`` twice when the first add decides at run time)."""

    def __init__(self, p, has_bias, layer_norm=None, dropout_mod=None):
        super().__init__()
        self.p = p
        self.has_bias = has_bias
        self.layer_norm = layer_norm
        # keep the original nn.Dropout (not called): its ``training`` flag follows
        # ``model.eval()`` like every other sub-module's
        self.dropout_mod = dropout_mod

    def forward(self, *args):
        if self.has_bias:
            x, bias = _split_bias(args[0], args[1])
            residual = args[2]
        else:
            x, bias, residual = args[0], None, args[1]
        training = self.training
        if self.layer_norm is None:
            return NF.bias_dropout_add(x, bias, residual, self.p, training)
        ln = self.layer_norm
        y, _ = NF.dropout_add_layer_norm(x, bias, residual, ln.weight, ln.bias, self.p, ln.eps,
                                         training)
        return y

    def extra_repr(self):
        return f"p={self.p}, bias={self.has_bias}, layer_norm={self.layer_norm is not None}"


def _check_residual_position(gm, nodes, has_bias):
    """The extracted graph's placeholders come in first-use order; the kernels
    take (x, bias, residual) - make sure the chain reads them in that order."""
    placeholders = [n for n in gm.graph.nodes if n.op == "placeholder"]
    want = 3 if has_bias else 2
    if len(placeholders) != want:
        raise NotImplementedError(
            f"the chain reads {len(placeholders)} outside values; the fused kernel takes {want}")
    second_add = nodes[2] if has_bias else nodes[1]
    if placeholders[-1] not in second_add.all_input_nodes:
        raise NotImplementedError("the residual must enter at the add after the dropout")


def build_native_module(sch, chain) -> nn.Module:
    """Module calling the fused sm_100a kernel for ``chain`` (a list of
    ``(parent_path, node)``), or ``NotImplementedError``."""
    gm = sch._construct_fx_graph(chain)
    nodes = [n for n in gm.graph.nodes if n.op not in ("placeholder", "output", "get_attr")]
    kinds, attrs = zip(*(_classify(gm, n) for n in nodes))
    kinds = list(kinds)
    if kinds == ["add", "act"]:
        return NativeBiasAct(attrs[1]["act"])
    ln = None
    if kinds and kinds[-1] == "layer_norm":
        if "module" not in attrs[-1]:
            raise NotImplementedError("a functional layer_norm cannot be fused; use nn.LayerNorm")
        ln = attrs[-1]["module"]
        if len(ln.normalized_shape) != 1 or not ln.elementwise_affine:
            raise NotImplementedError("only affine LayerNorm over the last axis is fused")
        kinds = kinds[:-1]
    if kinds in (["add", "dropout", "add"], ["dropout", "add"]):
        has_bias = len(kinds) == 3
        drop = attrs[1 if has_bias else 0]
        _check_residual_position(gm, nodes, has_bias)
        if drop.get("training") is False:
            p = 0.0
        else:
            p = drop["p"]
        return NativeBiasDropoutAdd(p, has_bias, ln, drop.get("module"))
    raise NotImplementedError(
        "no native kernel for the chain " + " -> ".join(kinds + (["layer_norm"] if ln else [])))
