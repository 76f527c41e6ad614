"""Cross entropy, plain and vocabulary-parallel.

Each tensor-parallel rank holds the logits of its own vocabulary range
``[rank*V/p, (rank+1)*V/p)``.  The loss needs three group-wide quantities per
token - the row maximum, the sum of exponentials and the logit of the target.
On CUDA one streaming kernel (``ce_stats``) produces the three local numbers
per row without materialising an fp32 copy of the logits, they are combined
over the group with one MAX and one packed SUM all-reduce (nothing on a single
GPU), and a second kernel (``ce_grad``) writes ``softmax - onehot`` directly
in the logits' dtype.  Rows whose label equals ``ignore_index`` are neither
read nor do they contribute.  On CPU the same algebra runs in PyTorch.

Returns the per-token loss (no reduction), like the reference.

Parity: slapo/op/cross_entropy.py:17-158 of the reference.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from . import native


LOCAL = "local"  # sentinel group: the logits are not sharded, never communicate


def _group_info(group):
    if isinstance(group, str) and group == LOCAL:
        return 1, 0
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


class _VocabParallelCrossEntropy(torch.autograd.Function):
    """PyTorch implementation (CPU ranks, odd shapes, label smoothing)."""

    @staticmethod
    def forward(ctx, logits, target, group, label_smoothing=0.0, ignore_index=-100):
        world, rank = _group_info(group)
        part = logits.shape[-1]
        lo = rank * part
        lf = logits.float()
        row_max = lf.max(dim=-1).values
        if world > 1:
            dist.all_reduce(row_max, op=dist.ReduceOp.MAX, group=group)
        lf = lf - row_max.unsqueeze(-1)
        ignored = target == ignore_index
        outside = (target < lo) | (target >= lo + part) | ignored
        local_t = (target - lo).masked_fill(outside, 0)
        picked = lf.gather(-1, local_t.unsqueeze(-1)).squeeze(-1).masked_fill(outside, 0.0)
        exp = lf.exp()
        packed = torch.stack([picked, exp.sum(dim=-1)], dim=0)
        if label_smoothing > 0:
            packed = torch.cat([packed, lf.sum(dim=-1).unsqueeze(0)], dim=0)
        if world > 1:
            dist.all_reduce(packed, group=group)
        picked, sum_exp = packed[0], packed[1]
        loss = sum_exp.log() - picked
        softmax = exp / sum_exp.unsqueeze(-1)
        vocab = part * world
        if label_smoothing > 0:
            mean_logp = packed[2] / vocab - sum_exp.log()
            loss = (1.0 - label_smoothing) * loss - label_smoothing * mean_logp
        loss = loss.masked_fill(ignored, 0.0)
        ctx.label_smoothing, ctx.vocab = label_smoothing, vocab
        ctx.save_for_backward(softmax.to(logits.dtype), outside, local_t, ignored)
        return loss

    @staticmethod
    def backward(ctx, grad):
        softmax, outside, local_t, ignored = ctx.saved_tensors
        g = softmax.float()
        onehot_scale = (~outside).float() * (1.0 - ctx.label_smoothing)
        g.scatter_add_(-1, local_t.unsqueeze(-1), -onehot_scale.unsqueeze(-1))
        if ctx.label_smoothing > 0:
            g -= ctx.label_smoothing / ctx.vocab
        g *= grad.masked_fill(ignored, 0.0).unsqueeze(-1)
        return g.to(softmax.dtype), None, None, None, None


class _FusedCrossEntropy(torch.autograd.Function):
    """CUDA path on the ``ce_stats`` / ``ce_grad`` kernels."""

    @staticmethod
    def forward(ctx, logits, target, group, ignore_index):
        world, rank = _group_info(group)
        shape = target.shape
        logits2 = logits.reshape(-1, logits.shape[-1])
        target1 = target.reshape(-1).contiguous()
        lo = rank * logits2.shape[-1]
        stats = native.ops().ce_stats(logits2, target1, lo, ignore_index)
        row_max, sum_exp, picked = stats[:, 0], stats[:, 1], stats[:, 2]
        if world > 1:
            gmax = row_max.clone()
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
            scale = torch.where(row_max == float("-inf"), torch.zeros_like(row_max),
                                (row_max - gmax).exp())
            packed = torch.stack([sum_exp * scale, picked], dim=0)
            dist.all_reduce(packed, group=group)
            sum_exp, picked, row_max = packed[0], packed[1], gmax
        valid = target1 != ignore_index
        lse = torch.where(valid, row_max + sum_exp.log(), torch.zeros_like(row_max))
        loss = torch.where(valid, lse - picked, torch.zeros_like(lse))
        ctx.save_for_backward(logits2, target1, lse)
        ctx.lo, ctx.ignore_index, ctx.logits_shape = lo, ignore_index, logits.shape
        return loss.view(shape)

    @staticmethod
    def backward(ctx, grad):
        logits2, target1, lse = ctx.saved_tensors
        coef = grad.reshape(-1).float().contiguous()
        g = native.ops().ce_grad(logits2, target1, lse, coef, ctx.lo, ctx.ignore_index)
        return g.view(ctx.logits_shape), None, None, None


def _fused_ok(logits, label_smoothing):
    return (logits.is_cuda and label_smoothing == 0.0 and logits.shape[-1] % 8 == 0
            and logits.dtype in (torch.bfloat16, torch.float16, torch.float32)
            and logits.is_contiguous() and native.available())


def vocab_parallel_cross_entropy(logits, target, group=None, label_smoothing=0.0,
                                 ignore_index=-100):
    """Per-token cross entropy of (vocabulary-sharded) ``logits``; tokens with
    ``target == ignore_index`` get loss 0 and no gradient."""
    if _fused_ok(logits, label_smoothing):
        return _FusedCrossEntropy.apply(logits, target, group, ignore_index)
    return _VocabParallelCrossEntropy.apply(logits, target, group, label_smoothing, ignore_index)


def cross_entropy(logits, target, ignore_index=-100):
    """Single-device fused cross entropy (per token)."""
    return vocab_parallel_cross_entropy(logits, target, LOCAL, 0.0, ignore_index)


class ParallelCrossEntropy(nn.Module):
    def __init__(self, group=None, label_smoothing=0.0, ignore_index=-100):
        super().__init__()
        self.group = group
        self.label_smoothing = label_smoothing
        self.ignore_index = ignore_index

    def forward(self, outputs, labels):
        return vocab_parallel_cross_entropy(outputs, labels, self.group, self.label_smoothing,
                                            self.ignore_index)
