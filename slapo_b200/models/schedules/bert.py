"""Scheduling recipes for BERT, RoBERTa.

``apply_schedule(model, "bert", model_config=cfg, ...)`` recognised options:

=====================  =====================================================
``model_config``       the model's config object (required)
``prefix``             path of the ``BertModel`` inside ``model`` ("bert")
``fp16`` / ``bf16``    cast the model
``group``              tensor-parallel process group
``attn_op_name``       attention kernel ("auto" = tcgen05 flash attention on
                       CUDA, PyTorch elsewhere; "reference" = PyTorch)
``disable_flash_attn`` keep the model's own attention
``fuse``               fuse bias+GeLU and bias+dropout+residual+LayerNorm
                       (default True)
``sequence_parallel``  shard the LN/dropout regions over the tokens
``sequence_parallel_axis``  which activation axis is split there: 0 = batch
                       (whole sequences per rank; the layout the fused
                       all-gather/reduce-scatter GEMMs take), 1 = sequence
``ckpt_ratio``         fraction of layers to checkpoint (0 = none)
``checkpoint_method``  "uniform" (spread) or "head" (first layers)
``bcast_input``        broadcast rank-0 inputs inside the TP group
``pipeline_cuts``      layer indices after which a pipeline stage ends
``trace_config``       for an unmodified Hugging Face model under pipeline cuts: the
                       example shapes its graphs are specialised on
                       (``{"batch_size": ..., "seq_len": ...}`` or ``input_shapes``)
``delay_init``         unused here (the caller decides to build on meta)
=====================  =====================================================

Parity: slapo/model_schedule/bert.py:18-342 and roberta.py:8-14 of the
reference.
"""
from __future__ import annotations

from torch import nn

from ... import create_schedule
from ...model_schedule.registry import register_schedule
from ...ops.attention import FlashAttention
from ...ops.blocks import FusedIntermediateBlock, FusedOutputBlock
from .common import (annotate_replicated, broadcast_input, cast_dtype, checkpoint_layers,
                     logger, shard_column, shard_row, shard_word_embedding, tracer_for)


class SelfAttentionAdapter(nn.Module):
    """Presents ``FlashAttention`` under HF's ``BertSelfAttention`` call
    convention; the child is named ``self_attn`` like in the reference."""

    def __init__(self, attn: FlashAttention):
        super().__init__()
        self.self_attn = attn

    def forward(self, hidden_states, attention_mask=None, **kwargs):
        return self.self_attn(hidden_states, attention_mask)


def _j(prefix, rest):
    return f"{prefix}.{rest}" if prefix else rest


def _layer_paths(sch, prefix):
    n = len([k for k in sch[_j(prefix, "encoder")].child if k.startswith("layer.")])
    return [_j(prefix, f"encoder.layer.{i}") for i in range(n)]


def replace_attention(sch, config, prefix, attn_op_name):
    count = 0
    for path in _layer_paths(sch, prefix):
        sub = sch[f"{path}.attention.self"]
        old = sub.mod
        if isinstance(old, SelfAttentionAdapter):
            continue
        attn = FlashAttention(
            config.hidden_size, config.num_attention_heads,
            attn_pdrop=config.attention_probs_dropout_prob, attn_op_name=attn_op_name,
            output_proj=False, fused_qkv=True, causal=False, device="meta")
        w, b = old.query.weight, old.query.bias
        if not w.is_meta:
            attn.qkv.weight = nn.Parameter(FlashAttention.layout_qkv_from_separate(
                old.query.weight.data, old.key.weight.data, old.value.weight.data,
                config.num_attention_heads))
            attn.qkv.bias = nn.Parameter(FlashAttention.layout_qkv_from_separate(
                old.query.bias.data, old.key.bias.data, old.value.bias.data,
                config.num_attention_heads))
        else:
            attn.qkv.weight = nn.Parameter(w.new_empty((3 * w.shape[0], w.shape[1])))
            attn.qkv.bias = nn.Parameter(b.new_empty((3 * b.shape[0],)))
        sub.replace(SelfAttentionAdapter(attn))
        count += 1
    return count


def fuse_blocks(sch, config, prefix):
    count = 0
    p = config.hidden_dropout_prob
    for path in _layer_paths(sch, prefix):
        for name in ("attention.output", "output"):
            sub = sch[f"{path}.{name}"]
            if not isinstance(sub.mod, FusedOutputBlock):
                sub.replace(FusedOutputBlock(sub.mod.dense, sub.mod.LayerNorm, p))
                count += 1
        sub = sch[f"{path}.intermediate"]
        if not isinstance(sub.mod, FusedIntermediateBlock):
            sub.replace(FusedIntermediateBlock(sub.mod.dense, config.hidden_act))
            count += 1
    return count


def shard_layers(sch, config, prefix, sequence_parallel, sp_axis=0, pipeline=False):
    if sch.world_size == 1:
        return 0
    if config.num_attention_heads % sch.world_size != 0:
        raise ValueError(f"{config.num_attention_heads} heads cannot be split over "
                         f"{sch.world_size} ranks")
    for path in _layer_paths(sch, prefix):
        attn = sch[f"{path}.attention.self"]
        if isinstance(attn.mod, SelfAttentionAdapter):
            shard_column(attn["self_attn.qkv"], sequence_parallel=sequence_parallel, sp_axis=sp_axis)
            if not sequence_parallel and config.attention_probs_dropout_prob > 0:
                attn["self_attn.attn_op"].fork_rng()
        else:
            for name in ("query", "key", "value"):
                shard_column(attn[name], sequence_parallel=sequence_parallel, sp_axis=sp_axis)
        shard_row(sch[f"{path}.attention.output.dense"], sequence_parallel, sp_axis)
        shard_column(sch[f"{path}.intermediate.dense"], sequence_parallel=sequence_parallel,
                     sp_axis=sp_axis)
        shard_row(sch[f"{path}.output.dense"], sequence_parallel, sp_axis)
        if sequence_parallel:
            annotate_replicated(
                sch, [f"{path}.attention.output.LayerNorm", f"{path}.output.LayerNorm"],
                [f"{path}.attention.output.dense", f"{path}.output.dense"])
    if sequence_parallel:
        # the embedding block computes the full sequence on every rank; keep
        # this rank's part, and put the sequence together again after the
        # last layer (the consumers are replicas, so the gradient is sliced)
        sch[_j(prefix, "embeddings")].sync("fwd_post", "scatter", axis=sp_axis)
        # With pipeline cuts the encoder dissolves into the stages and a hook on it would be
        # lost: the gather then sits on the last layer, which stays a module of the last stage.
        end = _layer_paths(sch, prefix)[-1] if pipeline else _j(prefix, "encoder")
        sch[end].sync("fwd_post", "all_gather", axis=sp_axis, tensor_parallel_output_grad=False)
    return len(_layer_paths(sch, prefix))


def shard_lm_head(sch, config, prefix):
    """Vocabulary-parallel embedding + tied decoder.  The logits stay sharded
    along the vocabulary; use ``mlm_loss(..., vocab_parallel=True)``."""
    if sch.world_size == 1:
        return
    shard_word_embedding(sch[_j(prefix, "embeddings.word_embeddings")], config.vocab_size)
    # BERT keeps the head under cls.predictions, RoBERTa under lm_head; same members
    head_path = "cls.predictions" if "cls.predictions" in sch else ("lm_head" if "lm_head" in sch else None)
    if head_path is not None:
        head = sch[head_path]
        head["decoder"].shard("weight", axis=0)  # tied: same shard as the embedding
        head["decoder"].shard("bias", axis=0)
        head.shard("bias", axis=0)               # the same Parameter under its second name
        head["decoder"].sync("bwd_post", "all_reduce")


def pipeline_cut(sch, prefix, cuts, trace_config=None):
    sch.trace_until(_j(prefix, "encoder"), tracer=tracer_for(sch.mod), config=trace_config)
    for idx in cuts:
        sch[_j(prefix, f"encoder.layer.{idx}")].cut_pipeline_stage()


@register_schedule("bert")
def schedule_bert(model, model_config=None, prefix="bert", fp16=False, bf16=False, group=None,
                  attn_op_name="auto", disable_flash_attn=False, fuse=True,
                  sequence_parallel=False, sequence_parallel_axis=0, ckpt_ratio=0.0,
                  checkpoint_method="uniform",
                  bcast_input=False, pipeline_cuts=None, shard_vocab=True, delay_init=True,
                  trace_config=None, **_unused):
    config = model_config if model_config is not None else getattr(model, "config", None)
    if config is None:
        raise ValueError("model_config is required")
    cast_dtype(model, fp16, bf16)
    sch = create_schedule(model, group=group)
    if prefix and prefix not in sch:
        prefix = ""
    pre = prefix
    n_attn = 0 if disable_flash_attn else replace_attention(sch, config, pre, attn_op_name)
    n_fused = fuse_blocks(sch, config, pre) if fuse else 0
    n_shard = shard_layers(sch, config, pre, sequence_parallel, sequence_parallel_axis,
                           pipeline=bool(pipeline_cuts))
    if shard_vocab and config.vocab_size % max(sch.world_size, 1) == 0:
        shard_lm_head(sch, config, pre)
    if bcast_input:
        broadcast_input(sch)
    n_ckpt = checkpoint_layers(sch, _layer_paths(sch, pre), ckpt_ratio, checkpoint_method)
    if pipeline_cuts:
        pipeline_cut(sch, pre, pipeline_cuts, trace_config)
    logger.info("bert schedule: %d attention replaced, %d blocks fused, %d layers sharded "
                "(sp=%s), %d checkpointed", n_attn, n_fused, n_shard, sequence_parallel, n_ckpt,
                ranks=0)
    return sch


@register_schedule("roberta")
def schedule_roberta(model, **kwargs):
    kwargs.setdefault("prefix", "roberta" if hasattr(model, "roberta") else "bert")
    return schedule_bert(model, **kwargs)
