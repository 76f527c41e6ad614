"""Activation-layout resharding over the last two dimensions.

A layout is written with two letters for the last two dimensions of an
activation ``[..., s, h]``: ``R`` = replicated, ``S`` = sharded over the
tensor-parallel group.  ``"RS"`` therefore means "hidden dimension sharded",
``"SR"`` "sequence dimension sharded".  ``reshard("RS->SR", x, group)``
moves between layouts; the nine schemes and their per-rank traffic (V =
bytes of the full tensor, p = group size) are

==========  =========================  =================
scheme      operation                  bytes received
==========  =========================  =================
RR->RS/SR   local slice                0
RS->RR      all-gather (last dim)      (p-1)/p * V
SR->RR      all-gather (dim -2)        (p-1)/p * V
RS->SR      all-to-all                 (p-1)/p^2 * V
SR->RS      all-to-all                 (p-1)/p^2 * V
XX->XX      identity                   0
==========  =========================  =================

Unlike the reference (slapo/sharding/reshard_ops.py:27-175, forward only)
every scheme is an autograd function: the gradient of a reshard is the
reverse reshard, which makes Ulysses-style head/sequence swaps trainable.
On a backend without all-to-all (gloo) the exchange is emulated with an
all-gather so that CPU ranks can act as the oracle.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .sync_ops import _world, all_gather_along_dim, scatter_along_dim

RESHARD_COST = {
    "RR->RS": lambda v, p: 0.0,
    "RR->SR": lambda v, p: 0.0,
    "RS->RR": lambda v, p: (p - 1) / p * v,
    "SR->RR": lambda v, p: (p - 1) / p * v,
    "RS->SR": lambda v, p: (p - 1) / p**2 * v,
    "SR->RS": lambda v, p: (p - 1) / p**2 * v,
    "RR->RR": lambda v, p: 0.0,
    "RS->RS": lambda v, p: 0.0,
    "SR->SR": lambda v, p: 0.0,
}

_AXIS = {"RS": -1, "SR": -2}

# process group (or None for the default group) -> FusedAllToAll
_FUSED_A2A = {}


def enable_fused_all_to_all(group, ctx):
    """Route the ``RS <-> SR`` all-to-all of ``group`` through the peer-store kernel over the
    symmetric-memory context ``ctx`` (collective: every rank of the group calls it)."""
    from .fused_a2a import FusedAllToAll

    _FUSED_A2A[group] = FusedAllToAll(ctx)
    return _FUSED_A2A[group]


def _all_to_all_dims(inp, split_dim, cat_dim, group):
    """Split ``inp`` along split_dim into p pieces, send piece j to rank j,
    concatenate what arrives along cat_dim."""
    world, rank = _world(group)
    if world == 1:
        return inp
    ndim = inp.dim()
    split_dim, cat_dim = split_dim % ndim, cat_dim % ndim
    fused = _FUSED_A2A.get(group)
    if fused is not None:
        inp_c = inp.contiguous()
        if fused.supports(inp_c, split_dim, cat_dim, world):
            return fused(inp_c, split_dim, cat_dim)
    pieces = [c.contiguous() for c in inp.chunk(world, dim=split_dim)]
    backend = dist.get_backend(group)
    if backend == "gloo":
        full = all_gather_along_dim(torch.stack(pieces, 0), 0, world, group)
        full = full.view((world, world) + tuple(pieces[0].shape))
        recv = [full[src, rank] for src in range(world)]
    else:
        recv = [torch.empty_like(pieces[0]) for _ in range(world)]
        dist.all_to_all(recv, pieces, group=group)
    return torch.cat(recv, dim=cat_dim)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, split_dim, cat_dim, group):
        ctx.split_dim, ctx.cat_dim, ctx.group = split_dim, cat_dim, group
        return _all_to_all_dims(inp, split_dim, cat_dim, group)

    @staticmethod
    def backward(ctx, grad):
        return _all_to_all_dims(grad, ctx.cat_dim, ctx.split_dim, ctx.group), None, None, None


class _GatherReplicated(torch.autograd.Function):
    """all-gather whose consumers are replicas: gradient = local slice."""

    @staticmethod
    def forward(ctx, inp, dim, group):
        ctx.dim, ctx.group = dim, group
        ctx.world = _world(group)[0]
        return all_gather_along_dim(inp, dim, ctx.world, group)

    @staticmethod
    def backward(ctx, grad):
        return scatter_along_dim(grad, ctx.dim, ctx.world, ctx.group), None, None


class _SliceReplicated(torch.autograd.Function):
    """local slice of a replicated tensor: gradient = all-gather."""

    @staticmethod
    def forward(ctx, inp, dim, group):
        ctx.dim, ctx.group = dim, group
        ctx.world = _world(group)[0]
        return scatter_along_dim(inp, dim, ctx.world, group)

    @staticmethod
    def backward(ctx, grad):
        return all_gather_along_dim(grad, ctx.dim, ctx.world, ctx.group), None, None


def reshard_RR_to_RS(inp, group=None):
    return _SliceReplicated.apply(inp, -1, group)


def reshard_RR_to_SR(inp, group=None):
    return _SliceReplicated.apply(inp, -2, group)


def reshard_RS_to_RR(inp, group=None):
    return _GatherReplicated.apply(inp, -1, group)


def reshard_SR_to_RR(inp, group=None):
    return _GatherReplicated.apply(inp, -2, group)


def reshard_RS_to_SR(inp, group=None):
    # hidden-sharded -> sequence-sharded: split the sequence, gather the hidden
    return _AllToAll.apply(inp, -2, -1, group)


def reshard_SR_to_RS(inp, group=None):
    return _AllToAll.apply(inp, -1, -2, group)


def _identity(inp, group=None):
    return inp


_TABLE = {
    "RR->RS": reshard_RR_to_RS, "RR->SR": reshard_RR_to_SR,
    "RS->RR": reshard_RS_to_RR, "SR->RR": reshard_SR_to_RR,
    "RS->SR": reshard_RS_to_SR, "SR->RS": reshard_SR_to_RS,
    "RR->RR": _identity, "RS->RS": _identity, "SR->SR": _identity,
}


def parse_reshard(scheme: str, group=None):
    """``"RS->SR"`` -> a function of the tensor."""
    key = scheme.replace(" ", "")
    if key not in _TABLE:
        raise ValueError(f"unknown reshard scheme '{scheme}' (use two letters R/S per side)")
    fn = _TABLE[key]
    return lambda inp: fn(inp, group)


def reshard(scheme: str, inp, group=None):
    return parse_reshard(scheme, group)(inp)
