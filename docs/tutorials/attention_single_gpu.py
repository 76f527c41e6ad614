"""Optimise a self-attention block on one device
================================================

    python docs/tutorials/attention_single_gpu.py

The block below is the textbook formulation: three separate projections, a materialised
``[B, H, S, S]`` score matrix, softmax, dropout, a fourth projection, bias + dropout +
residual + LayerNorm.  Step by step the schedule turns it into what this framework trains
BERT with - without editing the class:

1. trace the block into a graph (only this block; the rest of a model would stay eager);
2. find the three parallel projections with a pattern and fuse them *horizontally* into one
   GEMM whose output is laid out ``[head][q|k|v][dim]``;
3. find the core attention sub-graph and replace it *vertically* by the flash-attention
   operator (tcgen05 kernels on CUDA, a PyTorch reference on CPU);
4. fuse the tail (bias + dropout + residual + LayerNorm) into one kernel.

Every step is checked against the original block with ``Verify``-style comparisons.
"""
import copy
import math
import os
import sys

import torch
import torch.nn.functional as F
from torch import nn

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import slapo_b200 as slapo  # noqa: E402
from slapo_b200.ops import functional as NF  # noqa: E402
from slapo_b200.ops.attention import FlashAttentionOp  # noqa: E402
from slapo_b200.pattern import call_module  # noqa: E402

HIDDEN, HEADS = 64, 4


class SelfAttention(nn.Module):
    def __init__(self):
        super().__init__()
        self.query = nn.Linear(HIDDEN, HIDDEN)
        self.key = nn.Linear(HIDDEN, HIDDEN)
        self.value = nn.Linear(HIDDEN, HIDDEN)

    def split(self, t):
        return t.view(t.shape[0], t.shape[1], HEADS, HIDDEN // HEADS).permute(0, 2, 1, 3)

    def forward(self, x):
        q, k, v = self.split(self.query(x)), self.split(self.key(x)), self.split(self.value(x))
        scores = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(HIDDEN // HEADS)
        probs = F.softmax(scores, dim=-1)
        ctx = torch.matmul(probs, v).permute(0, 2, 1, 3)
        return ctx.reshape(ctx.shape[0], ctx.shape[1], HIDDEN)


class Output(nn.Module):
    def __init__(self):
        super().__init__()
        self.dense = nn.Linear(HIDDEN, HIDDEN)
        self.dropout = nn.Dropout(0.0)
        self.LayerNorm = nn.LayerNorm(HIDDEN)

    def forward(self, hidden, residual):
        return self.LayerNorm(self.dropout(self.dense(hidden)) + residual)


class Attention(nn.Module):
    def __init__(self):
        super().__init__()
        self.self = SelfAttention()
        self.output = Output()

    def forward(self, x):
        return self.output(self.self(x), x)


class FusedQKV(nn.Module):
    """One GEMM for q, k and v; rows ordered [head][q|k|v][dim] so that a tensor-parallel split
    of axis 0 would hand each rank whole heads."""

    def __init__(self, q, k, v):
        super().__init__()
        self.fused = nn.Linear(HIDDEN, 3 * HIDDEN)
        pack = lambda a, b, c: torch.cat(  # noqa: E731
            [t.reshape(HEADS, HIDDEN // HEADS, *t.shape[1:]) for t in (a, b, c)], dim=1
        ).reshape(-1, *a.shape[1:])
        with torch.no_grad():
            self.fused.weight.copy_(pack(q.weight, k.weight, v.weight))
            self.fused.bias.copy_(pack(q.bias, k.bias, v.bias))

    def forward(self, x):
        qkv = self.fused(x).view(x.shape[0], x.shape[1], HEADS, 3, HIDDEN // HEADS)
        # q, k, v as [B, S, H, D] views of the one projection output
        return qkv[..., 0, :], qkv[..., 1, :], qkv[..., 2, :]


class CoreAttention(nn.Module):
    """[B, S, H, D] q, k, v -> [B, S, H * D] context through the flash-attention operator."""

    def __init__(self):
        super().__init__()
        self.op = FlashAttentionOp(attn_op_name="auto", apply_causal_mask=False)

    def forward(self, q, k, v):
        ctx = self.op(q, k, v, None, 0.0)
        return ctx.reshape(ctx.shape[0], ctx.shape[1], -1)


class FusedTail(nn.Module):
    """dense -> (bias + dropout + residual + LayerNorm in one kernel)."""

    def __init__(self, out: Output):
        super().__init__()
        self.dense, self.LayerNorm, self.p = out.dense, out.LayerNorm, out.dropout.p

    def forward(self, hidden, residual):
        y, _ = NF.dropout_add_layer_norm(
            F.linear(hidden, self.dense.weight), self.dense.bias, residual,
            self.LayerNorm.weight, self.LayerNorm.bias, self.p, self.LayerNorm.eps, self.training)
        return y


def main():
    torch.manual_seed(0)
    block = Attention()
    original = copy.deepcopy(block)       # kept aside for the comparisons
    x = torch.randn(2, 16, HIDDEN)
    want = original(x)

    sch = slapo.create_schedule(block)
    # 1. static graph of the self-attention only; `split` is inlined by the tracer
    attn = sch["self"]
    attn.trace(flatten=True)
    print(attn.mod.graph)

    # 2. horizontal fusion: three matches, one replacement module, three outputs
    matches = attn.find(lambda t: call_module(r"query|key|value", t))
    assert len(matches) == 3
    qkv = FusedQKV(block.self.query, block.self.key, block.self.value)
    # 3. the whole attention becomes "fused projection, then the flash operator"

    class Scheduled(nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv, self.core = qkv, CoreAttention()

        def forward(self, t):
            return self.core(*self.qkv(t))

    attn.replace(Scheduled())
    torch.testing.assert_close(sch.mod(x), want, rtol=1e-4, atol=1e-4)

    # 4. the tail of the block
    sch["output"].replace(FusedTail(block.output))
    built, _ = slapo.build(sch, init_weights=False)
    torch.testing.assert_close(built(x), want, rtol=1e-4, atol=1e-4)
    # gradients agree as well
    xr = x.clone().requires_grad_(True)
    xs = x.clone().requires_grad_(True)
    original(xr).sum().backward()
    built(xs).sum().backward()
    torch.testing.assert_close(xs.grad, xr.grad, rtol=1e-4, atol=1e-4)
    print(built)
    print("attention tutorial finished")


if __name__ == "__main__":
    main()
