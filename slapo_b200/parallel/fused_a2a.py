"""All-to-all of the ``RS <-> SR`` activation reshards as one peer-store kernel.

``FusedAllToAll(ctx)(x, split_dim, cat_dim)`` is the drop-in for "chunk along
``split_dim``, exchange, concatenate along ``cat_dim``" on the last two
dimensions of a contiguous activation: every rank stores block ``j`` of its
tensor straight into rank ``j``'s receive buffer (symmetric memory, NVLink)
at the place the concatenation wants it, so there is no packing copy before
and no ``cat`` after the exchange; the kernel ends with a bounded handshake.
Receive buffers alternate between two symmetric allocations, which makes the
result safe to read while peers already run the next exchange.  The reference
implements the same reshard with ``permute -> chunk -> dist.all_to_all -> cat
-> permute`` on NCCL, forward only (slapo/sharding/reshard_ops.py:107-175).
"""
from __future__ import annotations

import torch

from ..ops import native


class FusedAllToAll:
    def __init__(self, ctx, wait_seconds=None):
        self.ctx = ctx
        self.wait_seconds = wait_seconds if wait_seconds is not None else ctx.wait_seconds
        self.calls = 0
        self.flag_buf = ctx.buffer("a2a_flags", 8 * 4)
        self.counter = torch.zeros(1, dtype=torch.int32, device=ctx.device)

    @staticmethod
    def supports(inp, split_dim, cat_dim, world):
        nd = inp.dim()
        if nd < 2 or not inp.is_cuda or not inp.is_contiguous():
            return False
        s, c = split_dim % nd, cat_dim % nd
        if {s, c} != {nd - 1, nd - 2}:
            return False
        if inp.shape[s] % world:
            return False
        esize = inp.element_size()
        row = inp.shape[-1] * esize if s == nd - 2 else inp.shape[-1] // world * esize
        return row % 16 == 0

    def push(self, inp, split_dim, cat_dim):
        """Launch the exchange; returns this rank's receive view (complete once every rank's
        kernel has run)."""
        ctx, p, rank = self.ctx, self.ctx.world, self.ctx.rank
        nd = inp.dim()
        s = split_dim % nd
        e = inp.element_size()
        outer = 1
        for d in inp.shape[:-2]:
            outer *= d
        if s == nd - 2:          # RS -> SR: split the rows, concatenate the columns
            S, hl = inp.shape[-2], inp.shape[-1]
            sl = S // p
            rows, row_bytes = sl, hl * e
            src = (sl * hl * e, S * hl * e, hl * e)
            dst = (rank * hl * e, sl * hl * p * e, hl * p * e)
            out_shape = tuple(inp.shape[:-2]) + (sl, hl * p)
        else:                    # SR -> RS: split the columns, concatenate the rows
            sl, h = inp.shape[-2], inp.shape[-1]
            hl = h // p
            rows, row_bytes = sl, hl * e
            src = (hl * e, sl * h * e, h * e)
            dst = (rank * sl * hl * e, sl * p * hl * e, hl * e)
            out_shape = tuple(inp.shape[:-2]) + (sl * p, hl)
        nbytes = inp.numel() * e
        name = f"a2a_recv_{self.calls % 2}"
        self.calls += 1
        recv = ctx.buffer(name, nbytes)
        epoch = ctx.next_epoch()
        native.ops().peer_all_to_all(
            inp, recv.ptrs(), self.flag_buf.ptrs(), p, rank, epoch, outer, rows, row_bytes,
            src[0], src[1], src[2], dst[0], dst[1], dst[2], self.counter, self.wait_seconds)
        return recv.view(inp.dtype, out_shape)

    def __call__(self, inp, split_dim, cat_dim):
        return self.push(inp, split_dim, cat_dim).clone()
