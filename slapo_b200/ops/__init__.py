"""Modules and functions that schedules swap into models."""
from .linear import (FusedQKV, LinearWithAct, LinearWithDropout,  # noqa: F401
                     LinearWithSeparateBias, LinearWithSyncFunc)
from .attention import FlashAttention, FlashAttentionOp  # noqa: F401
from .cross_entropy import ParallelCrossEntropy  # noqa: F401
from .mlp import FusedMLP  # noqa: F401
from .norm import FusedDropoutAddLayerNorm, FusedLayerNorm, FusedRMSNorm  # noqa: F401
from .utils import Print  # noqa: F401
