"""Vocabulary-parallel cross entropy.

Each tensor-parallel rank holds the logits of its own vocabulary range
``[rank*V/p, (rank+1)*V/p)``.  The loss needs three group-wide quantities per
token - the row maximum, the logit of the target and the sum of
exponentials - so the local pass produces them and they are exchanged with
three small all-reduces (MAX, SUM, SUM; the latter two are packed into one
message here).  The backward is ``softmax - onehot`` on the local slice.

Returns the per-token loss (no reduction), like the reference.

Parity: slapo/op/cross_entropy.py:17-158 of the reference.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn


def _group_info(group):
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


class _VocabParallelCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, group, label_smoothing=0.0):
        world, rank = _group_info(group)
        part = logits.shape[-1]
        lo = rank * part
        lf = logits.float()
        row_max = lf.max(dim=-1).values
        if world > 1:
            dist.all_reduce(row_max, op=dist.ReduceOp.MAX, group=group)
        lf = lf - row_max.unsqueeze(-1)
        outside = (target < lo) | (target >= lo + part)
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
            # smoothed target = (1-a) onehot + a/V
            mean_logp = packed[2] / vocab - sum_exp.log()
            loss = (1.0 - label_smoothing) * loss - label_smoothing * mean_logp
        ctx.label_smoothing, ctx.vocab = label_smoothing, vocab
        ctx.save_for_backward(softmax.to(logits.dtype), outside, local_t)
        return loss

    @staticmethod
    def backward(ctx, grad):
        softmax, outside, local_t = ctx.saved_tensors
        g = softmax.float()
        onehot_scale = (~outside).float() * (1.0 - ctx.label_smoothing)
        g.scatter_add_(-1, local_t.unsqueeze(-1), -onehot_scale.unsqueeze(-1))
        if ctx.label_smoothing > 0:
            g -= ctx.label_smoothing / ctx.vocab
        g *= grad.unsqueeze(-1)
        return g.to(softmax.dtype), None, None, None


def vocab_parallel_cross_entropy(logits, target, group=None, label_smoothing=0.0):
    return _VocabParallelCrossEntropy.apply(logits, target, group, label_smoothing)


class ParallelCrossEntropy(nn.Module):
    def __init__(self, group=None, label_smoothing=0.0):
        super().__init__()
        self.group = group
        self.label_smoothing = label_smoothing

    def forward(self, outputs, labels):
        return vocab_parallel_cross_entropy(outputs, labels, self.group, self.label_smoothing)
