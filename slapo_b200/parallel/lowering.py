"""Lower ``shard`` + ``sync`` pairs to fused GEMM+collective kernels.

The schedule primitives describe tensor parallelism as "a sharded Linear plus
a collective next to it" (hooks and ``sync_fn``), which runs anywhere through
``torch.distributed``.  On a B200 node :func:`lower_fused_tp` rewrites every
pair it recognises so that the collective happens *inside* the GEMM kernel
over NVLink peer memory (see csrc/comm_gemm.cu):

=============================================  ==============================
schedule                                       fused plan on the Linear
=============================================  ==============================
``sync("fwd_pre", "all_gather", axis=0)``      ``fused_pre = ("ag", ctx)``
``sync("fwd_post", "reduce_scatter", axis=0)`` ``fused_post = ("rs", ctx)``
``sync("fwd_post", "all_reduce")``             ``fused_post = ("ar", ctx)``
``sync("bwd_post", "all_reduce")``             ``fused_bwd = ("ar", ctx)``
=============================================  ==============================

Anything else (other axes, custom hooks, non-Linear modules) keeps its
``torch.distributed`` hook.  The reference does the analogous module swap for
row-parallel layers only (slapo/sharding/shard_ops.py:497-519) and always calls
NCCL.
"""
from __future__ import annotations

from torch import nn

from ..logger import get_logger
from ..ops.linear import LinearWithSyncFunc
from .shard_methods import SyncFn, SyncHook

logger = get_logger("lowering")


def _pop_sync_hook(mod, op, **match):
    for key, hook in list(mod._forward_pre_hooks.items()):
        if isinstance(hook, SyncHook) and hook.op == op and all(
                hook.kwargs.get(k, d) == v for k, (v, d) in match.items()):
            del mod._forward_pre_hooks[key]
            return hook
    return None


def _lower_vocab_embedding(sub, ctx) -> bool:
    """``shard_word_embedding`` (masked lookup + all-reduce / reduce-scatter hooks) -> the
    peer-store kernel, in its all-gather form or - under sequence parallelism - its scatter
    form.  16-bit weights only."""
    import torch

    from ..ops.embedding import FusedVocabParallelEmbedding

    mod = sub.mod
    hooks = getattr(mod, "_vocab_parallel_hooks", None)
    if hooks is None or mod.weight.is_meta:
        return False
    if hooks.sequence_parallel and hooks.sp_axis not in (0, 1):
        return False
    if mod.weight.dtype not in (torch.bfloat16, torch.float16) or mod.embedding_dim % 8:
        return False
    for table in (mod._forward_pre_hooks, mod._forward_hooks):
        for key, fn in list(table.items()):
            if getattr(fn, "__self__", None) is hooks:
                del table[key]
    sub.replace(FusedVocabParallelEmbedding.from_sharded(
        mod, sub.rank, ctx, hooks.sp_axis if hooks.sequence_parallel else None))
    return True


def lower_fused_tp(sch, ctx) -> int:
    """Attach fused plans below schedule ``sch``; returns how many Linears changed."""
    changed = 0
    for _, sub in list(sch.named_schedules()):
        mod = sub.mod
        if isinstance(mod, nn.Embedding):
            if _lower_vocab_embedding(sub, ctx):
                logger.info("lowered %s to the peer-store vocabulary-parallel embedding",
                            sub.path, ranks=0)
            continue
        if not isinstance(mod, nn.Linear):
            continue
        pre_ag = _pop_sync_hook(mod, "all_gather", axis=(0, 0),
                                tensor_parallel_output_grad=(True, True))
        bwd_ar = None if pre_ag else _pop_sync_hook(mod, "bwd_all_reduce")
        post = None
        fn = getattr(mod, "sync_fn", None)
        if isinstance(fn, SyncFn):
            if fn.sync_op == "reduce_scatter" and fn.sync_kwargs.get("axis", 0) == 0:
                post = "rs"
            elif fn.sync_op == "all_reduce":
                post = "ar"
        if not (pre_ag or bwd_ar or post):
            continue
        if (pre_ag or post) and (mod.weight.shape[0] % 8 or mod.weight.shape[1] % 8):
            # rows of 16-bit operands must be multiples of 16 bytes for TMA: put the hooks back
            raise ValueError(
                f"{sub.path}: the fused tensor-parallel kernels need weight shards whose "
                f"dimensions are multiples of 8, got {tuple(mod.weight.shape)}")
        if not isinstance(mod, LinearWithSyncFunc):
            new = LinearWithSyncFunc.from_linear(mod)
            sub.replace(new)
            mod = new
        if pre_ag:
            mod.fused_pre = ("ag", ctx)
        if bwd_ar:
            mod.fused_bwd = ("ar", ctx)
        if post:
            mod.fused_post = (post, ctx)
            mod.sync_fn = None
        changed += 1
    logger.info("lowered %d sharded Linear layers to fused GEMM+collective kernels", changed,
                ranks=0)
    return changed
