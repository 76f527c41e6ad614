"""Scheduling recipe for ALBERT: the single shared layer group is scheduled
once and every depth benefits.  q / k / v and ``ffn`` column-parallel,
``attention.dense`` and ``ffn_output`` row-parallel, the factorised word
embedding vocabulary-parallel, bias + activation of ``ffn`` fused.

``pipeline_cuts=[k, ...]`` ends a stage after the k-th pass (0-based) through
the layers: the encoder is traced, which unrolls its loop into one call of
the shared group per pass, and the cut is put on that call.  Every stage
holds the shared layer; the pipeline engine ties the copies.  (The reference
cuts at ``encoder.layer.k``, a path that ALBERT models do not have -
slapo/model_schedule/albert.py:118-141.)

Parity: slapo/model_schedule/albert.py:21-353 of the reference.
"""
from __future__ import annotations

from ... import create_schedule
from ...model_schedule.registry import register_schedule
from ...ops.linear import LinearWithAct
from .common import (broadcast_input, cast_dtype, logger, shard_column, shard_row,
                     shard_word_embedding, tracer_for)


def _layers(sch, prefix):
    out = []
    enc = sch[f"{prefix}.encoder"]
    for g in [k for k in enc.child if k.startswith("albert_layer_groups.")]:
        grp = enc[g]
        for l in [k for k in grp.child if k.startswith("albert_layers.")]:
            out.append(f"{prefix}.encoder.{g}.{l}")
    return out


def pipeline_cut(sch, config, prefix, cuts, trace_config=None):
    """End a stage after pass ``k`` through the layers, for every ``k`` in ``cuts``."""
    sch.trace_until(f"{prefix}.encoder", tracer=tracer_for(sch.mod), config=trace_config)
    per_group = config.num_hidden_layers // config.num_hidden_groups
    for k in cuts:
        if not 0 <= k < config.num_hidden_layers - 1:
            raise ValueError(f"pipeline cut {k}: the model makes {config.num_hidden_layers} "
                             "passes, a stage can end after pass 0 .. "
                             f"{config.num_hidden_layers - 2}")
        group = sch[f"{prefix}.encoder.albert_layer_groups.{k // per_group}"]
        group.cut_pipeline_stage(call_index=k % per_group)


@register_schedule("albert")
def schedule_albert(model, model_config=None, prefix="albert", fp16=False, bf16=False,
                    group=None, fuse=True, ckpt_ratio=0.0, bcast_input=False, pipeline_cuts=None,
                    trace_config=None, **_unused):
    config = model_config if model_config is not None else getattr(model, "config", None)
    if config is None:
        raise ValueError("model_config is required")
    cast_dtype(model, fp16, bf16)
    sch = create_schedule(model, group=group)
    layers = _layers(sch, prefix)
    for path in layers:
        if fuse:
            ffn = sch[f"{path}.ffn"]
            ffn.replace(LinearWithAct.from_linear(ffn.mod, act_fn=config.hidden_act))
            # the activation module after it becomes the identity
            sch[f"{path}.activation"].replace(__import__("torch").nn.Identity())
        if sch.world_size > 1:
            for name in ("query", "key", "value"):
                shard_column(sch[f"{path}.attention.{name}"])
            shard_row(sch[f"{path}.attention.dense"])
            shard_column(sch[f"{path}.ffn"])
            shard_row(sch[f"{path}.ffn_output"])
    if sch.world_size > 1 and config.vocab_size % sch.world_size == 0:
        shard_word_embedding(sch[f"{prefix}.embeddings.word_embeddings"], config.vocab_size)
        if "predictions" in sch:
            head = sch["predictions"]
            head["decoder"].shard("weight", axis=0)
            head["decoder"].shard("bias", axis=0)
            head.shard("bias", axis=0)
            head["decoder"].sync("bwd_post", "all_reduce")
    if bcast_input:
        broadcast_input(sch)
    if ckpt_ratio > 0:
        for path in layers:
            sch[path].checkpoint()
    if pipeline_cuts:
        pipeline_cut(sch, config, prefix, pipeline_cuts, trace_config)
    logger.info("albert schedule: %d shared layers scheduled (tp=%d)", len(layers),
                sch.world_size, ranks=0)
    return sch
