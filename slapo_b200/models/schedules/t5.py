"""Scheduling recipe for T5 (encoder-decoder, relative-position bias, plain or
gated feed-forward).

Projection fusion (``fuse_qkv``, default on): self-attention q / k / v become one
``qkv`` GEMM, cross-attention k / v one ``kv`` GEMM (:class:`T5FusedAttention`).

Tensor parallelism: the (fused) projections column-parallel (whole heads per rank), ``o``
row-parallel, the relative-position table split along its head axis, ``wi``
(or the gate pair ``wi_0`` / ``wi_1``, split identically) column-parallel,
``wo`` row-parallel, the shared embedding vocabulary-parallel with the tied
``lm_head``.  The reference needs the external ``epoi`` package for T5
attention and asserts gated feed-forwards away
(slapo/model_schedule/t5.py:211-265, :463); here attention is the in-tree
flash kernel with in-line bias lookup and gated FFNs shard like plain ones.

Pipeline cuts: ``pipeline_cuts=[enc_cuts, dec_cuts]``; the encoder itself
always ends a stage when any cut is given, so that the tail of the encoder
never fuses with the head of the decoder.

Parity: slapo/model_schedule/t5.py:19-489 of the reference.
"""
from __future__ import annotations

from ... import create_schedule
from ...model_schedule.registry import register_schedule
from .common import (broadcast_input, cast_dtype, checkpoint_layers, logger,
                     shard_word_embedding, tracer_for)


def _blocks(sch, stack):
    n = len([k for k in sch[stack].child if k.startswith("block.")])
    return [f"{stack}.block.{i}" for i in range(n)]


def fuse_projections(sch):
    """Replace every attention module by its fused-projection form; returns how many."""
    from ..t5 import T5Attention, T5FusedAttention

    count = 0
    for stack in ("encoder", "decoder"):
        for blk in _blocks(sch, stack):
            paths = [(f"{blk}.layer.0.SelfAttention", False)]
            if stack == "decoder":
                paths.append((f"{blk}.layer.1.EncDecAttention", True))
            for path, cross in paths:
                if isinstance(sch[path].mod, T5Attention):
                    sch[path].replace(T5FusedAttention(sch[path].mod, cross))
                    count += 1
    return count


def _shard_attention(sch, path):
    names = [n for n in ("qkv", "kv", "q", "k", "v") if n in sch[path].child]
    for name in names:
        sch[f"{path}.{name}"].shard("weight", axis=0)
        sch[f"{path}.{name}"].sync("bwd_post", "all_reduce")
    sch[f"{path}.o"].shard("weight", axis=1)
    sch[f"{path}.o"].sync("fwd_post", "all_reduce")
    if "relative_attention_bias" in sch[path].child:
        sch[f"{path}.relative_attention_bias"].shard("weight", axis=1)


def _shard_ffn(sch, path, gated):
    names = ("wi_0", "wi_1") if gated else ("wi",)
    for name in names:
        sch[f"{path}.{name}"].shard("weight", axis=0)
        sch[f"{path}.{name}"].sync("bwd_post", "all_reduce")
    sch[f"{path}.wo"].shard("weight", axis=1)
    sch[f"{path}.wo"].sync("fwd_post", "all_reduce")


def shard_t5(sch, config):
    if sch.world_size == 1:
        return 0
    if config.num_heads % sch.world_size:
        raise ValueError(f"{config.num_heads} heads cannot be split over {sch.world_size} ranks")
    count = 0
    for stack in ("encoder", "decoder"):
        for blk in _blocks(sch, stack):
            _shard_attention(sch, f"{blk}.layer.0.SelfAttention")
            if stack == "decoder":
                _shard_attention(sch, f"{blk}.layer.1.EncDecAttention")
            ff = f"{blk}.layer.2" if stack == "decoder" else f"{blk}.layer.1"
            _shard_ffn(sch, f"{ff}.DenseReluDense", config.is_gated_act)
            count += 1
    if config.vocab_size % sch.world_size == 0:
        # Hugging Face's T5 (recent versions) gives each stack an embedding module of its own
        # that shares the weight of ``shared``: every module that looks tokens up needs the
        # vocabulary-parallel hooks, and ``shard`` keeps the one tensor tied among them
        seen = set()
        for path in ("shared", "encoder.embed_tokens", "decoder.embed_tokens"):
            if path in sch and id(sch[path].mod) not in seen:
                seen.add(id(sch[path].mod))
                shard_word_embedding(sch[path], config.vocab_size)
        sch["lm_head"].shard("weight", axis=0)
        sch["lm_head"].sync("bwd_post", "all_reduce")
    return count


@register_schedule("t5")
def schedule_t5(model, model_config=None, fp16=False, bf16=False, group=None, ckpt_ratio=0.0,
                checkpoint_method="uniform", bcast_input=False, pipeline_cuts=None, trace_config=None,
                fuse_qkv=True, **_unused):
    config = model_config if model_config is not None else getattr(model, "config", None)
    if config is None:
        raise ValueError("model_config is required")
    cast_dtype(model, fp16, bf16)
    sch = create_schedule(model, group=group)
    n_fused = fuse_projections(sch) if fuse_qkv else 0
    n_shard = shard_t5(sch, config)
    if bcast_input:
        broadcast_input(sch)
    n_ckpt = 0
    for stack in ("encoder", "decoder"):
        n_ckpt += checkpoint_layers(sch, _blocks(sch, stack), ckpt_ratio, checkpoint_method)
    if pipeline_cuts:
        enc_cuts, dec_cuts = pipeline_cuts
        sch.trace_until(["encoder", "decoder"], tracer=tracer_for(sch.mod), config=trace_config)
        for idx in enc_cuts:
            sch[f"encoder.block.{idx}"].cut_pipeline_stage()
        sch["encoder"].cut_pipeline_stage()
        for idx in dec_cuts:
            sch[f"decoder.block.{idx}"].cut_pipeline_stage()
    logger.info("t5 schedule: %d attention modules with fused projections, %d blocks sharded, "
                "%d checkpointed", n_fused, n_shard, n_ckpt, ranks=0)
    return sch
