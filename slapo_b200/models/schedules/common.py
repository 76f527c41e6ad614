"""Building blocks shared by the per-model scheduling recipes."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ...logger import get_logger
from ...parallel.sync_ops import reduce_forward_output, reduce_scatter_forward_output

logger = get_logger("model_schedule")


def cast_dtype(model, fp16=False, bf16=False):
    if fp16 and bf16:
        raise ValueError("fp16 and bf16 are exclusive")
    if fp16:
        model.half()
    elif bf16:
        model.bfloat16()
    return model


def shard_column(sch, names=("weight", "bias"), sequence_parallel=False, sp_axis=1):
    """Column-parallel Linear: split the output features; the input gradient
    is a partial sum, so it is all-reduced (or, under sequence parallelism,
    the input is all-gathered and its gradient reduce-scattered)."""
    for name in names:
        if getattr(sch.mod, name, None) is not None:
            sch.shard(name, axis=0)
    if sequence_parallel:
        sch.sync("fwd_pre", "all_gather", axis=sp_axis)
    else:
        sch.sync("bwd_post", "all_reduce")


def shard_row(sch, sequence_parallel=False, sp_axis=1):
    """Row-parallel Linear: split the input features; the output is a partial
    sum that is all-reduced (or reduce-scattered along the sequence)."""
    sch.shard("weight", axis=1)
    if sequence_parallel:
        sch.sync("fwd_post", "reduce_scatter", axis=sp_axis)
    else:
        sch.sync("fwd_post", "all_reduce")


class VocabParallelEmbeddingHooks:
    """Forward hooks turning a row-sharded ``nn.Embedding`` into a
    vocabulary-parallel one.

    The pre-hook shifts the ids into the local range and remembers which ids
    belong to other ranks; the post-hook zeroes *exactly those* rows and sums
    over the group (all-reduce, or reduce-scatter along the sequence under
    sequence parallelism).  The mask is carried from the pre-hook to the
    post-hook - recomputing it from the already shifted ids, as the
    reference's BERT/OPT/T5 recipes do (slapo/model_schedule/bert.py:263-280),
    zeroes the wrong rows."""

    def __init__(self, sch, sequence_parallel=False, sp_axis=1):
        self.group = sch.group
        self.world = sch.world_size
        self.rank = sch.rank
        self.sequence_parallel = sequence_parallel
        self.sp_axis = sp_axis
        self._mask = None

    def __deepcopy__(self, memo):
        return self

    def pre(self, module, inputs):
        ids = inputs[0]
        lo = self.rank * module.num_embeddings
        outside = (ids < lo) | (ids >= lo + module.num_embeddings)
        self._mask = outside
        return ((ids - lo).masked_fill(outside, 0),) + tuple(inputs[1:])

    def meta_shape(self, shape):
        """Output shape after the post-hook (see ``SyncHook.meta_shape``)."""
        out = list(shape)
        if self.sequence_parallel and len(out) > self.sp_axis:
            out[self.sp_axis] //= self.world
        return tuple(out)

    def post(self, module, inputs, output):
        output = output.masked_fill(self._mask.unsqueeze(-1), 0.0)
        self._mask = None
        if self.sequence_parallel:
            return reduce_scatter_forward_output(output, self.sp_axis, self.group)
        return reduce_forward_output(output, self.group)


def shard_word_embedding(sch, vocab_size, sequence_parallel=False, sp_axis=1):
    """Vocabulary-parallel word embedding (the tied LM head follows).  Under
    sequence parallelism the partial lookups are reduce-scattered along
    ``sp_axis`` instead of all-reduced."""
    if sch.world_size == 1:
        return
    if vocab_size % sch.world_size != 0:
        raise ValueError(f"vocab size {vocab_size} must be padded to a multiple of "
                         f"{sch.world_size} before sharding")
    sch.shard("weight", axis=0)
    hooks = VocabParallelEmbeddingHooks(sch, sequence_parallel, sp_axis)
    sch.sync("fwd_pre", hooks.pre)
    sch.sync("fwd_post", hooks.post)
    # lets the lowering pass recognise the pair and swap in the peer-store kernel
    sch.mod._vocab_parallel_hooks = hooks


def checkpoint_layers(sch, layer_paths, ckpt_ratio, method="uniform", order_args_fn=None):
    """Checkpoint ``ckpt_ratio`` of the layers: ``"head"`` = the first
    ``int(L*r)`` layers, ``"uniform"`` = spread evenly over the depth."""
    n = len(layer_paths)
    if ckpt_ratio <= 0 or n == 0:
        return 0
    config = getattr(sch.get_top_schedule().mod, "config", None)
    if getattr(config, "use_cache", False):
        # A recomputed layer runs twice; a key / value cache that the model threads through
        # its layers (Hugging Face models build one when ``use_cache`` is on) would be
        # appended to twice.  Hugging Face's own gradient checkpointing switches it off too.
        config.use_cache = False
        logger.info("use_cache is switched off: activation checkpointing runs layers twice",
                    ranks=0)
    n_ckpt = int(n * min(ckpt_ratio, 1.0))
    if method == "head":
        chosen = list(range(n_ckpt))
    else:
        chosen = sorted({int(i * n / n_ckpt) for i in range(n_ckpt)}) if n_ckpt else []
    for idx in chosen:
        sch[layer_paths[idx]].checkpoint(order_args_fn=order_args_fn)
    return len(chosen)


def broadcast_input(sch):
    """Make every TP rank consume rank 0's inputs."""
    if sch.world_size == 1:
        return
    group = sch.group
    src = dist.get_global_rank(group, 0) if group is not None else 0

    def hook(_module, inputs):
        for t in inputs:
            if torch.is_tensor(t):
                dist.broadcast(t, src=src, group=group)
        return inputs

    sch.sync("fwd_pre", hook)


def annotate_replicated(sch, layer_norm_paths=(), bias_paths=()):
    """Tag parameters that are replicated over the TP group but see only a
    sequence shard of the activations: their gradients must be summed over
    the group (the engine does it for ``replicated_param`` tensors)."""
    for path in layer_norm_paths:
        for name in ("weight", "bias"):
            if getattr(sch[path].mod, name, None) is not None:
                sch[path].annotate(name, "replicated_param", True)
    for path in bias_paths:
        if getattr(sch[path].mod, "bias", None) is not None:
            sch[path].annotate("bias", "replicated_param", True)


def tracer_for(model):
    """Tracer name for ``trace_until`` in a recipe's pipeline cut: unmodified Hugging Face
    models need the ``"huggingface"`` tracer (meta-tensor shapes, ``ModelOutput`` reads,
    catch-all keyword arguments); this package's own models trace with plain ``"pytorch"``."""
    try:
        from transformers import PreTrainedModel
    except Exception:  # transformers is optional
        return "pytorch"
    return "huggingface" if isinstance(model, PreTrainedModel) else "pytorch"


def pad_vocab(vocab_size, multiple):
    return (vocab_size + multiple - 1) // multiple * multiple
