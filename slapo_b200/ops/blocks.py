"""Fused transformer sub-blocks used by the model schedules.

They keep the child names of the Hugging Face blocks they replace
(``dense`` / ``LayerNorm`` / ``dropout``), so parameter paths - and with them
``shard`` calls, checkpoints and ``Verify`` - are unchanged, while the forward
runs ``matmul -> [collective] -> one kernel for bias + dropout + residual +
LayerNorm``.
"""
from __future__ import annotations

from torch import nn

from . import functional as NF
from .linear import LinearWithAct, LinearWithSyncFunc


class FusedOutputBlock(nn.Module):
    """``LayerNorm(dropout(dense(x)) + residual)`` - BERT's ``BertSelfOutput``
    and ``BertOutput`` - with the tail fused."""

    def __init__(self, dense: nn.Linear, layer_norm: nn.LayerNorm, p: float):
        super().__init__()
        self.dense = dense if isinstance(dense, LinearWithSyncFunc) \
            else LinearWithSyncFunc.from_linear(dense)
        self.LayerNorm = layer_norm
        self.dropout = nn.Dropout(p)

    def forward(self, hidden_states, input_tensor):
        out = self.dense(hidden_states, skip_bias=True)
        y, _ = NF.dropout_add_layer_norm(
            out, self.dense.bias, input_tensor, self.LayerNorm.weight, self.LayerNorm.bias,
            self.dropout.p, self.LayerNorm.eps, self.training)
        return y


class FusedIntermediateBlock(nn.Module):
    """``act(dense(x))`` - BERT's ``BertIntermediate`` - with bias + activation fused."""

    def __init__(self, dense: nn.Linear, act_name: str):
        super().__init__()
        self.dense = dense if isinstance(dense, LinearWithAct) \
            else LinearWithAct.from_linear(dense, act_fn=act_name)

    def forward(self, hidden_states):
        return self.dense(hidden_states)
