"""Normalisation modules backed by the fused sm_100a kernels.

* ``FusedLayerNorm`` / ``FusedRMSNorm`` - drop-in for ``nn.LayerNorm`` /
  T5 layer norm;
* ``FusedDropoutAddLayerNorm`` - ``LayerNorm(dropout(x + bias) + residual)``
  in one pass (the pattern the reference fuses with TorchScript in
  tests/test_fusion.py:157-204).
"""
import torch
from torch import nn

from . import functional as NF


class FusedLayerNorm(nn.LayerNorm):
    def forward(self, x):
        return NF.layer_norm(x, self.weight, self.bias, self.eps)


class FusedRMSNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-6, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.variance_epsilon = eps

    def forward(self, x):
        return NF.rms_norm(x, self.weight, self.variance_epsilon)


class FusedDropoutAddLayerNorm(nn.Module):
    """``forward(x, residual, bias=None) -> LayerNorm(dropout(x + bias) + residual)``.

    With ``return_residual=True`` also returns the pre-norm sum."""

    def __init__(self, hidden_size, p=0.1, eps=1e-5, return_residual=False, device=None,
                 dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(hidden_size, device=device, dtype=dtype))
        self.p, self.eps, self.return_residual = p, eps, return_residual

    def forward(self, x, residual, bias=None):
        y, z = NF.dropout_add_layer_norm(x, bias, residual, self.weight, self.bias, self.p,
                                         self.eps, self.training)
        return (y, z) if self.return_residual else y
