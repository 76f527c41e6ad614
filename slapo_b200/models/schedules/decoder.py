"""Scheduling recipes for the decoder-only families: GPT-2, GPT-Neo, OPT.

One generic recipe, parameterised by a *layout* (where the blocks, attention,
MLP, embeddings and head live in each model).  Options (``sch_config``):
``model_config`` (required), ``prefix``, ``fp16`` / ``bf16``, ``group``,
``attn_op_name``, ``disable_flash_attn``, ``fuse`` (FusedMLP / fused
LayerNorm), ``sequence_parallel`` (+ ``sequence_parallel_axis``),
``ckpt_ratio``, ``checkpoint_method`` (``uniform`` | ``head``), ``bcast_input``,
``pipeline_cuts``, ``trace_config`` (the example shapes - ``batch_size``, ``seq_len`` or
``input_shapes`` - that the graphs of an unmodified Hugging Face model are specialised on when
pipeline cuts make the recipe trace it).

Tensor parallelism: fused QKV column-parallel (whole heads per rank),
attention output and MLP output row-parallel, vocabulary-parallel embedding
with the tied ``lm_head`` column-parallel over the vocabulary (use
``causal_lm_loss(..., vocab_parallel=True)``).  With sequence parallelism the
token dimension of the LayerNorm / dropout regions is split: scatter after
the embeddings, all-gather before the column-parallel layers, reduce-scatter
after the row-parallel ones, all-gather after ``ln_f``.

Parity: slapo/model_schedule/gpt2.py:19-661, gpt_neo.py:21-461,
opt.py:21-355 of the reference.  Differences on purpose: the OPT ``lm_head``
gets its missing gradient sync (reference opt.py:274-276 has none); heads that
do not divide the group size raise instead of silently mis-sharding.
"""
from __future__ import annotations

from torch import nn

from ... import create_schedule
from ...model_schedule.registry import register_schedule
from ...ops.attention import FlashAttention
from ...ops.mlp import FusedMLP
from ...ops.norm import FusedLayerNorm
from .common import (annotate_replicated, broadcast_input, cast_dtype, checkpoint_layers,
                     logger, shard_column, shard_row, shard_word_embedding, tracer_for)

LAYOUTS = {
    "gpt2": dict(prefix="transformer", layers="h", attn="attn", kind="conv1d_fused",
                 ln1="ln_1", ln2="ln_2", mlp="mlp", fc_in="c_fc", fc_out="c_proj",
                 wte="wte", pos=["wpe"], ln_f="ln_f", head="lm_head", scale=None,
                 heads="num_heads", act="activation_function", pdrop="resid_dropout",
                 attn_pdrop="attention_dropout", inter="intermediate_size"),
    "gpt_neo": dict(prefix="transformer", layers="h", attn="attn.attention", kind="separate",
                    ln1="ln_1", ln2="ln_2", mlp="mlp", fc_in="c_fc", fc_out="c_proj",
                    wte="wte", pos=["wpe"], ln_f="ln_f", head="lm_head", scale=1.0,
                    heads="num_heads", act="activation_function", pdrop="resid_dropout",
                    attn_pdrop="attention_dropout", inter="intermediate_size"),
    "opt": dict(prefix="model.decoder", layers="layers", attn="self_attn", kind="separate",
                ln1="self_attn_layer_norm", ln2="final_layer_norm", mlp=None, fc_in="fc1",
                fc_out="fc2", wte="embed_tokens", pos=["embed_positions"],
                ln_f="final_layer_norm", head="lm_head", scale=None,
                heads="num_attention_heads", act="activation_function", pdrop="dropout",
                attn_pdrop="attention_dropout", inter="ffn_dim"),
}


def _j(*parts):
    return ".".join(p for p in parts if p)


# the same field under the names of this library's configs and of Hugging Face's
_ALIASES = {
    "num_heads": ("num_heads", "num_attention_heads", "n_head"),
    "num_attention_heads": ("num_attention_heads", "num_heads", "n_head"),
    "resid_dropout": ("resid_dropout", "resid_pdrop"),
    "attention_dropout": ("attention_dropout", "attn_pdrop"),
    "intermediate_size": ("intermediate_size", "n_inner"),
}


def _cfg(config, key):
    """``config.<key>`` with the aliases above; a missing or ``None`` feed-forward width is
    four times the hidden size (the Hugging Face convention)."""
    for name in _ALIASES.get(key, (key,)):
        val = getattr(config, name, None)
        if val is not None:
            return val
    if key == "intermediate_size":
        return 4 * config.hidden_size
    raise AttributeError(f"the model configuration has none of {_ALIASES.get(key, (key,))}")


def _layer_paths(sch, lay, prefix):
    base = sch[prefix]
    n = len([k for k in base.child if k.startswith(lay["layers"] + ".")])
    return [_j(prefix, f"{lay['layers']}.{i}") for i in range(n)]


class AttentionAdapter(nn.Module):
    """Presents ``FlashAttention`` under the model's attention call
    convention ``(hidden_states, attention_mask) -> (output, None)``."""

    def __init__(self, attn):
        super().__init__()
        self.self_attn = attn

    def forward(self, hidden_states, attention_mask=None, **_ignored):
        return self.self_attn(hidden_states, attention_mask)


def _extract_qkv(old, kind, hidden):
    """(q, k, v) weights as [out, in] and biases (or None), (out_w, out_b)."""
    if kind == "conv1d_fused":
        w = old.c_attn.weight.data.t()  # [3h, in]
        b = old.c_attn.bias.data
        qw, kw, vw = w.chunk(3, dim=0)
        qb, kb, vb = b.chunk(3, dim=0)
        return (qw, kw, vw), (qb, kb, vb), (old.c_proj.weight.data.t(), old.c_proj.bias.data)
    ws = (old.q_proj.weight.data, old.k_proj.weight.data, old.v_proj.weight.data)
    bs = None
    if old.q_proj.bias is not None:
        bs = (old.q_proj.bias.data, old.k_proj.bias.data, old.v_proj.bias.data)
    return ws, bs, (old.out_proj.weight.data, old.out_proj.bias.data)


def replace_attention(sch, config, lay, prefix, attn_op_name):
    count = 0
    hidden = config.hidden_size
    heads = _cfg(config, lay["heads"])
    for path in _layer_paths(sch, lay, prefix):
        sub = sch[_j(path, lay["attn"])]
        old = sub.mod
        if isinstance(old, AttentionAdapter):
            continue
        probe = old.c_attn if lay["kind"] == "conv1d_fused" else old.q_proj
        has_bias = probe.bias is not None
        is_meta = probe.weight.is_meta
        attn = FlashAttention(hidden, heads, attn_pdrop=_cfg(config, lay["attn_pdrop"]),
                              resid_pdrop=_cfg(config, lay["pdrop"]) if lay["mlp"] else 0.0,
                              attn_op_name=attn_op_name, bias=has_bias, output_proj=True,
                              fused_qkv=True, causal=True, scale=lay["scale"],
                              device="meta" if is_meta else probe.weight.device,
                              dtype=probe.weight.dtype)
        if not is_meta:
            ws, bs, (ow, ob) = _extract_qkv(old, lay["kind"], hidden)
            attn.qkv.weight = nn.Parameter(
                FlashAttention.layout_qkv_from_separate(*[w.contiguous() for w in ws], heads))
            if bs is not None:
                attn.qkv.bias = nn.Parameter(FlashAttention.layout_qkv_from_separate(*bs, heads))
            attn.out_proj.weight = nn.Parameter(ow.contiguous())
            attn.out_proj.bias = nn.Parameter(ob.contiguous())
        sub.replace(AttentionAdapter(attn))
        count += 1
    return count


def replace_mlp(sch, config, lay, prefix):
    """GPT-style ``mlp`` blocks become ``FusedMLP`` (bias+activation and
    bias+dropout kernels); OPT keeps ``fc1`` / ``fc2`` at block level."""
    if lay["mlp"] is None:
        return 0
    count = 0
    for path in _layer_paths(sch, lay, prefix):
        sub = sch[_j(path, lay["mlp"])]
        old = sub.mod
        if isinstance(old, FusedMLP):
            continue
        fc_in, fc_out = getattr(old, lay["fc_in"]), getattr(old, lay["fc_out"])
        is_meta = fc_in.weight.is_meta
        new = FusedMLP(config.hidden_size, _cfg(config, lay["inter"]),
                       _cfg(config, lay["act"]), _cfg(config, lay["pdrop"]),
                       device="meta" if is_meta else fc_in.weight.device, dtype=fc_in.weight.dtype)
        if not is_meta:
            transposed = fc_in.weight.shape[0] == config.hidden_size and \
                fc_in.weight.shape[1] != config.hidden_size  # Conv1D stores [in, out]
            for dst, src in ((new.fc_in, fc_in), (new.fc_out, fc_out)):
                w = src.weight.data.t() if transposed else src.weight.data
                dst.weight = nn.Parameter(w.contiguous())
                dst.bias = nn.Parameter(src.bias.data.clone())
        sub.replace(new)
        count += 1
    return count


def replace_layernorm(sch):
    def make(name, mod):
        new = FusedLayerNorm(mod.normalized_shape, eps=mod.eps, device="meta")
        new.weight, new.bias = mod.weight, mod.bias
        return new

    targets = [(n, s) for n, s in sch.named_schedules()
               if type(s.mod) is nn.LayerNorm]
    for _, sub in targets:
        sub.replace(make("", sub.mod))
    return len(targets)


def shard_layers(sch, config, lay, prefix, sequence_parallel, sp_axis):
    if sch.world_size == 1:
        return 0
    heads = _cfg(config, lay["heads"])
    if heads % sch.world_size:
        raise ValueError(
            f"{heads} attention heads cannot be split over {sch.world_size} ranks; use a "
            "tensor-parallel size that divides the head count (e.g. TP 4 x DP 2 for 20 heads)")
    for path in _layer_paths(sch, lay, prefix):
        attn = sch[_j(path, lay["attn"])]
        if not isinstance(attn.mod, AttentionAdapter):
            raise RuntimeError("tensor parallelism needs the FlashAttention replacement "
                               "(disable_flash_attn=False)")
        shard_column(attn["self_attn.qkv"], sequence_parallel=sequence_parallel, sp_axis=sp_axis)
        shard_row(attn["self_attn.out_proj"], sequence_parallel, sp_axis)
        if not sequence_parallel:
            attn["self_attn.attn_op"].fork_rng()
        mlp_base = _j(path, lay["mlp"]) if lay["mlp"] else path
        fc_in = sch[_j(mlp_base, "fc_in" if lay["mlp"] else lay["fc_in"])]
        fc_out = sch[_j(mlp_base, "fc_out" if lay["mlp"] else lay["fc_out"])]
        shard_column(fc_in, sequence_parallel=sequence_parallel, sp_axis=sp_axis)
        shard_row(fc_out, sequence_parallel, sp_axis)
        if sequence_parallel:
            annotate_replicated(
                sch, [_j(path, lay["ln1"]), _j(path, lay["ln2"])],
                [_j(path, lay["attn"], "self_attn.out_proj"),
                 _j(mlp_base, "fc_out" if lay["mlp"] else lay["fc_out"])])
    if sequence_parallel and sp_axis == 1 and lay["mlp"] is None \
            and tracer_for(sch.mod) == "huggingface":
        raise ValueError(
            "Hugging Face's OPT layer flattens its tokens to [batch * sequence, hidden] in front "
            "of fc1, where a gather along the sequence axis has no meaning; use "
            "sequence_parallel_axis=0 (whole sequences per rank) for this model")
    if sequence_parallel and _positions_follow_embeddings(sch, sp_axis):
        # whole-sequence embeddings (the token table all-reduces), split where the first block
        # takes them over
        first = sch[_layer_paths(sch, lay, prefix)[0]]
        first.sync("fwd_pre", "scatter", axis=sp_axis)
        sch[_j(prefix, lay["ln_f"])].sync("fwd_post", "all_gather", axis=sp_axis,
                                          tensor_parallel_output_grad=False)
        annotate_replicated(sch, [_j(prefix, lay["ln_f"])], [])
    elif sequence_parallel:
        wte_meta = sch[_j(prefix, lay["wte"])].metadata.primitives.get("shard") or {}
        if "weight" not in wte_meta:  # a vocabulary-parallel embedding reduce-scatters itself
            sch[_j(prefix, lay["wte"])].sync("fwd_post", "scatter", axis=sp_axis)
        for pos in lay["pos"]:
            if sp_axis == 1:  # position embeddings are [1, S, H]: only a sequence split applies
                sch[_j(prefix, pos)].sync("fwd_post", "scatter", axis=sp_axis)
            else:
                # under a batch split every rank adds the whole [1, S, H] table to its own
                # sequences, so the table's gradient is a partial sum like a LayerNorm's
                sch[_j(prefix, pos)].annotate("weight", "replicated_param", True)
        sch[_j(prefix, lay["ln_f"])].sync("fwd_post", "all_gather", axis=sp_axis,
                                          tensor_parallel_output_grad=False)
        annotate_replicated(sch, [_j(prefix, lay["ln_f"])], [])
    return len(_layer_paths(sch, lay, prefix))


def _positions_follow_embeddings(sch, sp_axis):
    """Hugging Face decoders (recent ``transformers``) number the positions from the length of
    the embedded tokens.  With the sequence axis split inside the embedding, every rank would
    count from zero over its own part; for those models the embeddings stay whole and the
    split happens in front of the first block."""
    return sp_axis == 1 and tracer_for(sch.mod) == "huggingface"


def shard_embedding_and_head(sch, config, lay, prefix, sequence_parallel, sp_axis=1):
    if sch.world_size == 1 or config.vocab_size % sch.world_size:
        return
    wte = sch[_j(prefix, lay["wte"])]
    if sequence_parallel and _positions_follow_embeddings(sch, sp_axis):
        sequence_parallel = False
    shard_word_embedding(wte, config.vocab_size, sequence_parallel, sp_axis)
    if lay["head"] in sch:
        head = sch[lay["head"]]
        head.shard("weight", axis=0)  # tied with the embedding: same shard
        head.sync("bwd_post", "all_reduce")


def schedule_decoder(model, family, model_config=None, prefix=None, fp16=False, bf16=False,
                     group=None, attn_op_name="auto", disable_flash_attn=False, fuse=True,
                     sequence_parallel=False, sequence_parallel_axis=1, ckpt_ratio=0.0,
                     checkpoint_method="uniform", bcast_input=False, pipeline_cuts=None,
                     trace_config=None,
                     shard_vocab=True, **_unused):
    lay = LAYOUTS[family]
    config = model_config if model_config is not None else getattr(model, "config", None)
    if config is None:
        raise ValueError("model_config is required")
    cast_dtype(model, fp16, bf16)
    sch = create_schedule(model, group=group)
    prefix = lay["prefix"] if prefix is None else prefix
    if prefix not in sch:  # the trunk itself was passed in
        prefix = prefix.split(".", 1)[1] if "." in prefix and prefix.split(".", 1)[1] in sch else ""
    n_attn = 0 if disable_flash_attn else replace_attention(sch, config, lay, prefix, attn_op_name)
    n_mlp = replace_mlp(sch, config, lay, prefix) if fuse else 0
    n_ln = replace_layernorm(sch) if fuse else 0
    if shard_vocab:
        shard_embedding_and_head(sch, config, lay, prefix, sequence_parallel,
                                 sequence_parallel_axis)
    n_shard = shard_layers(sch, config, lay, prefix, sequence_parallel, sequence_parallel_axis)
    if bcast_input:
        broadcast_input(sch)
    n_ckpt = checkpoint_layers(sch, _layer_paths(sch, lay, prefix), ckpt_ratio, checkpoint_method)
    if pipeline_cuts:
        sch.trace_until(prefix, tracer=tracer_for(sch.mod), config=trace_config)
        for idx in pipeline_cuts:
            sch[_j(prefix, f"{lay['layers']}.{idx}")].cut_pipeline_stage()
    logger.info("%s schedule: %d attention, %d MLP, %d LayerNorm replaced; %d layers sharded "
                "(sp=%s); %d checkpointed", family, n_attn, n_mlp, n_ln, n_shard,
                sequence_parallel, n_ckpt, ranks=0)
    return sch


@register_schedule("gpt2")
def schedule_gpt2(model, **kwargs):
    return schedule_decoder(model, "gpt2", **kwargs)


@register_schedule("gpt_neo")
def schedule_gpt_neo(model, **kwargs):
    return schedule_decoder(model, "gpt_neo", **kwargs)


@register_schedule("opt")
def schedule_opt(model, **kwargs):
    return schedule_decoder(model, "opt", **kwargs)
