"""Vocabulary-parallel embedding whose forward needs no all-reduce.

With the vocabulary split over the tensor-parallel group, exactly one rank
owns the row of every token id.  ``FusedVocabParallelEmbedding`` lets that
rank store the row directly into every rank's output over NVLink peer memory
(``csrc/dp_comm.cu: vocab_embed_fwd_kernel``) instead of "masked local lookup
+ all-reduce of mostly zeros".  The mask that decides ownership is computed
from the *original* ids inside the kernel - the reference's recipes recompute
it from already shifted ids and zero the wrong rows
(slapo/model_schedule/bert.py:263-280).  The backward is local: every rank
sees the full output gradient and accumulates the rows of the ids it owns.
"""
from __future__ import annotations

import torch
from torch import nn

from . import native


class _VocabEmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, mod):
        sctx = mod.symm_ctx
        flat = ids.reshape(-1).contiguous()
        hidden = weight.shape[1]
        nbytes = flat.numel() * hidden * weight.element_size()
        name = f"vocab_embed_out_{mod.calls % 2}"      # alternate: peers may run one call ahead
        mod.calls += 1
        out_buf = sctx.buffer(name, nbytes)
        native.ops().vocab_embed_fwd(flat, weight, out_buf.ptrs(), mod.flag_buf.ptrs(), sctx.world,
                                     sctx.rank, sctx.next_epoch(), mod.vocab_start_index,
                                     mod.cta_counter, sctx.wait_seconds)
        out = out_buf.view(weight.dtype, (flat.numel(), hidden)).clone()
        ctx.save_for_backward(flat)
        ctx.lo, ctx.rows, ctx.dtype = mod.vocab_start_index, weight.shape[0], weight.dtype
        return out.view(tuple(ids.shape) + (hidden,))

    @staticmethod
    def backward(ctx, grad):
        (flat,) = ctx.saved_tensors
        local = flat - ctx.lo
        own = (local >= 0) & (local < ctx.rows)
        g = grad.reshape(flat.numel(), -1)
        grad_w = torch.zeros(ctx.rows, g.shape[1], dtype=torch.float32, device=g.device)
        grad_w.index_add_(0, local[own], g[own].float())
        return None, grad_w.to(ctx.dtype), None


class FusedVocabParallelEmbedding(nn.Module):
    """Drop-in for a row-sharded ``nn.Embedding`` (``weight`` = this rank's
    ``[vocab / tp, hidden]`` slice) over a symmetric-memory context."""

    traceable = False

    def __init__(self, weight, vocab_start_index, symm_ctx, padding_idx=None):
        super().__init__()
        self.weight = weight
        self.vocab_start_index = int(vocab_start_index)
        self.num_embeddings, self.embedding_dim = weight.shape
        self.padding_idx = padding_idx
        self.symm_ctx = symm_ctx
        self.calls = 0
        self.flag_buf = symm_ctx.buffer("vocab_embed_flags", 8 * 4)
        self.cta_counter = torch.zeros(1, dtype=torch.int32, device=symm_ctx.device)

    @classmethod
    def from_sharded(cls, emb: nn.Embedding, rank, symm_ctx):
        lo = getattr(emb, "vocab_start_index", rank * emb.num_embeddings)
        return cls(emb.weight, lo, symm_ctx, emb.padding_idx)

    def forward(self, ids):
        return _VocabEmbedFn.apply(ids, self.weight, self)

    def extra_repr(self):
        return (f"{self.num_embeddings}, {self.embedding_dim}, vocab_start={self.vocab_start_index}, "
                "peer-store all-gather")
