"""NVTX ranges for timelines (Nsight Systems, ``torch.profiler``): named regions around the
phases of a training step and around the modules that schedule primitives created.

Ranges cost a few hundred nanoseconds each when no profiler listens, but they are still off
by default: ``enable(True)`` (or ``SLAPO_B200_NVTX=1`` in the environment, or
``EngineConfig(profile=True)``) switches them on.  On machines without CUDA every call is a
no-op.  The reference wraps the forward and backward of one step in ``record_function``
ranges (slapo/utils/report.py:43-60); this is the same idea for every step and every region.
"""
from __future__ import annotations

import contextlib
import os

import torch

_STATE = {"on": os.environ.get("SLAPO_B200_NVTX", "0") == "1"}


def enable(flag: bool = True):
    _STATE["on"] = bool(flag)


def enabled() -> bool:
    return _STATE["on"] and torch.cuda.is_available()


@contextlib.contextmanager
def range(name: str):   # noqa: A001 - mirrors torch.cuda.nvtx.range
    if not enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def annotate_modules(model: torch.nn.Module, classes=None, max_depth: int = 6) -> int:
    """Put a range named after the module path around the forward of every sub-module that
    is an instance of ``classes`` (default: the modules this library swaps in - fused blocks,
    attention, sharded linears, checkpoint wrappers) down to ``max_depth`` path components.
    Backward kernels inherit the names through autograd's sequence numbers in profilers that
    correlate them.  Returns the number of modules annotated; idempotent."""
    if classes is None:
        from ..ops.attention import FlashAttention
        from ..ops.blocks import FusedIntermediateBlock, FusedOutputBlock
        from ..ops.linear import LinearWithSyncFunc
        from ..primitives.checkpoint import CheckPointWrapper

        classes = (FlashAttention, FusedIntermediateBlock, FusedOutputBlock, LinearWithSyncFunc,
                   CheckPointWrapper)
    n = 0
    for path, mod in model.named_modules():
        if not path or path.count(".") >= max_depth or not isinstance(mod, classes):
            continue
        if getattr(mod, "_slapo_nvtx", False):
            continue
        label = f"{path} [{type(mod).__name__}]"

        def pre(_m, _a, _label=label):
            if enabled():
                torch.cuda.nvtx.range_push(_label)

        def post(_m, _a, _o):
            if enabled():
                torch.cuda.nvtx.range_pop()

        mod.register_forward_pre_hook(pre)
        mod.register_forward_hook(post)
        mod._slapo_nvtx = True
        n += 1
    return n
