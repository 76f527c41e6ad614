"""Equivalence table between ``torch.nn.functional`` calls and ``nn.Module``
classes, used by the sub-graph matcher so that a pattern written with
``F.relu`` also matches an ``nn.ReLU`` call.

Parity: slapo/utils/mapping.py:11-23 of the reference.
"""
import torch.nn.functional as F
from torch import nn

MAPPING_FROM_FUNCTIONAL_TO_MODULE = {
    F.embedding: nn.Embedding,
    F.layer_norm: nn.LayerNorm,
    F.dropout: nn.Dropout,
    F.group_norm: nn.GroupNorm,
    F.linear: nn.Linear,
    F.relu: nn.ReLU,
    F.gelu: nn.GELU,
    F.silu: nn.SiLU,
    F.tanh: nn.Tanh,
    F.softmax: nn.Softmax,
    F.conv1d: nn.Conv1d,
    F.conv2d: nn.Conv2d,
    F.batch_norm: nn.BatchNorm2d,
    F.mse_loss: nn.MSELoss,
    F.cross_entropy: nn.CrossEntropyLoss,
}
