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

Under sequence parallelism (``sp_axis`` 0 or 1) a rank keeps only its shard of
the tokens: the owner of a row stores it into that one rank (the
reduce-scatter of the recipe's hooks, slapo/model_schedule/gpt2.py:343-355 and
424-432 of the reference, without looking up or adding zeros).  The backward
first gathers the token-sharded output gradient with the peer-load gather
kernel, then accumulates locally as before.
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
        world = sctx.world
        scatter, seq, out_shape = 0, 0, tuple(ids.shape) + (hidden,)
        if mod.sp_axis is not None:
            if ids.dim() != 2 or ids.shape[mod.sp_axis] % world:
                raise ValueError(f"token ids {tuple(ids.shape)} cannot be split {world} ways "
                                 f"along axis {mod.sp_axis}")
            scatter, seq = (1, 0) if mod.sp_axis == 0 else (2, ids.shape[1])
            out_shape = ((ids.shape[0] // world, ids.shape[1], hidden) if mod.sp_axis == 0
                         else (ids.shape[0], ids.shape[1] // world, hidden))
        native.ops().vocab_embed_fwd(flat, weight, out_buf.ptrs(), mod.flag_buf.ptrs(), world,
                                     sctx.rank, sctx.next_epoch(), mod.vocab_start_index,
                                     mod.cta_counter, sctx.wait_seconds, scatter, seq)
        rows_out = flat.numel() // world if scatter else flat.numel()
        out = out_buf.view(weight.dtype, (rows_out, hidden)).clone()
        ctx.save_for_backward(flat)
        ctx.lo, ctx.rows, ctx.dtype = mod.vocab_start_index, weight.shape[0], weight.dtype
        ctx.sctx, ctx.sp_axis, ctx.ids_shape = sctx, mod.sp_axis, tuple(ids.shape)
        return out.view(out_shape)

    @staticmethod
    def backward(ctx, grad):
        (flat,) = ctx.saved_tensors
        local = flat - ctx.lo
        own = (local >= 0) & (local < ctx.rows)
        if ctx.sp_axis is not None:
            # every rank needs the gradient rows of the ids it owns, whoever kept the token
            from ..parallel.fused_tp import peer_gather

            world = ctx.sctx.world
            shard = grad.reshape(-1, grad.shape[-1]).contiguous()
            full = peer_gather(ctx.sctx, shard, "vocab_embed_grad")     # [world * rows, hidden]
            if ctx.sp_axis == 1:   # [world, B, S / world, H] -> [B, S, H]
                b, s = ctx.ids_shape
                full = full.view(world, b, s // world, -1).permute(1, 0, 2, 3)
            grad = full.reshape(flat.numel(), -1)
        g = grad.reshape(flat.numel(), -1)
        grad_w = torch.zeros(ctx.rows, g.shape[1], dtype=torch.float32, device=g.device)
        grad_w.index_add_(0, local[own], g[own].float())
        return None, grad_w.to(ctx.dtype), None


class FusedVocabParallelEmbedding(nn.Module):
    """Drop-in for a row-sharded ``nn.Embedding`` (``weight`` = this rank's
    ``[vocab / tp, hidden]`` slice) over a symmetric-memory context."""

    traceable = False

    def __init__(self, weight, vocab_start_index, symm_ctx, padding_idx=None, sp_axis=None):
        """``sp_axis``: None = every rank gets every token's row; 0 / 1 = sequence parallel,
        this rank keeps its chunk of the batch / of every sequence."""
        super().__init__()
        self.sp_axis = sp_axis
        self.weight = weight
        self.vocab_start_index = int(vocab_start_index)
        self.num_embeddings, self.embedding_dim = weight.shape
        self.padding_idx = padding_idx
        self.symm_ctx = symm_ctx
        self.calls = 0
        self.flag_buf = symm_ctx.buffer("vocab_embed_flags", 8 * 4)
        self.cta_counter = torch.zeros(1, dtype=torch.int32, device=symm_ctx.device)

    @classmethod
    def from_sharded(cls, emb: nn.Embedding, rank, symm_ctx, sp_axis=None):
        lo = getattr(emb, "vocab_start_index", rank * emb.num_embeddings)
        return cls(emb.weight, lo, symm_ctx, emb.padding_idx, sp_axis)

    def forward(self, ids):
        return _VocabEmbedFn.apply(ids, self.weight, self)

    def extra_repr(self):
        return (f"{self.num_embeddings}, {self.embedding_dim}, vocab_start={self.vocab_start_index}, "
                + ("peer-store all-gather" if self.sp_axis is None
                   else f"peer-store scatter along axis {self.sp_axis}"))
