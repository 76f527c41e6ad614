"""Fused two-layer MLP block.

``fc_in`` is a ``LinearWithAct`` (matmul, then one kernel for bias +
activation) and ``fc_out`` a ``LinearWithDropout`` (matmul, then one kernel
for bias + dropout).  The activation given by the caller is honoured (the
reference passes it into the wrong positional slot and always gets GeLU,
slapo/op/mlp.py:39).

Parity: slapo/op/mlp.py:10-50 of the reference.
"""
from torch import nn

from .linear import LinearWithAct, LinearWithDropout


class FusedMLP(nn.Module):
    def __init__(self, hidden_size, intermediate_size, orig_act="gelu", resid_pdrop=0.0,
                 use_torchscript=False, device=None, dtype=None):
        super().__init__()
        self.fc_in = LinearWithAct(hidden_size, intermediate_size, bias=True, act_fn=orig_act,
                                   device=device, dtype=dtype)
        self.fc_out = LinearWithDropout(intermediate_size, hidden_size, bias=True,
                                        p=resid_pdrop, device=device, dtype=dtype)

    def forward(self, hidden_states):
        return self.fc_out(self.fc_in(hidden_states))
