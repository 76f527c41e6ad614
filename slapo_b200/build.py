"""``build``: turn a schedule into a runnable (model, optimizer) pair.

Steps:

1. if any ``cut_pipeline_stage`` was applied, split the traced graphs into
   stage modules (:func:`generate_pipeline_partition`);
2. materialise delayed (meta-device) parameters consistently across the
   tensor-parallel group (``consolidate_model``);
3. with pipeline cuts, wrap the stages for the target runtime;
4. hand the model to the target's runtime engine.  ``target=None`` returns
   ``(model, None)``; ``target="native"`` returns this framework's training
   engine.

Consolidation: a sharded parameter remembers its full ``orig_shape``.  The
first rank of each group creates the full tensor and initialises it
(``init_weights(module[, path])``, the module's ``_init_weights`` or
``reset_parameters``), broadcasts it over the group, and every rank keeps
``chunk(world, axis)[rank]`` where ``axis`` is the one axis on which the
shapes differ - so a TP run starts from exactly the weights an unsharded run
with the same seed would have.  Works on CUDA (NCCL) and CPU (gloo).

Parity: slapo/build.py:28-272 of the reference (CUDA only there).
"""
from __future__ import annotations

import inspect

import torch
import torch.distributed as dist
from torch import nn

from .framework_dialect import get_dialect_cls
from .logger import get_logger
from .utils.common import transfor_param_tags

logger = get_logger("build")


def _default_device():
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def _shard_axis(full_shape, local_shape):
    diff = [i for i, (a, b) in enumerate(zip(full_shape, local_shape)) if a != b]
    if len(diff) > 1:
        raise RuntimeError(f"more than one sharded axis: {full_shape} -> {local_shape}")
    return diff[0] if diff else None


def _call_init(init_fn, mod, path):
    try:
        n_params = len(inspect.signature(init_fn).parameters)
    except (TypeError, ValueError):
        n_params = 1
    if n_params >= 2:
        init_fn(mod, path)
    else:
        init_fn(mod)


_UNTOUCHED_SEEN = set()


def _default_init_if_untouched(mod, names, init_fn):
    """Initialisers that dispatch on composite classes (Hugging Face's T5 fills the projections
    from ``T5Attention`` / ``T5DenseActDense``, the embedding from the model class) do nothing
    for the layer itself when modules are initialised one at a time: a weight matrix that is
    still all zeros after the call gets the layer's own ``reset_parameters`` instead, so that
    the model trains - with PyTorch's default scheme for that layer, which the log says once."""
    owner = getattr(init_fn, "__self__", None)
    if not hasattr(mod, "reset_parameters") or not any(
            c.__name__ == "PreTrainedModel" for c in type(owner).__mro__):
        return      # only for Hugging Face's class-dispatching initialisers: anyone else's
        #             zeros are taken as meant
    still_zero = [n for n in names if mod._parameters[n].dim() > 1
                  and not bool(mod._parameters[n].data.any())]
    if not still_zero:
        return
    mod.reset_parameters()
    key = type(mod).__name__
    if key not in _UNTOUCHED_SEEN:
        _UNTOUCHED_SEEN.add(key)
        logger.info("%s left the weights of %s modules untouched (it initialises them from a "
                    "parent class); PyTorch's default initialiser is used for them",
                    getattr(init_fn, "__qualname__", init_fn), key, ranks=0)


def _pick_init_fn(top_mod, init_weights):
    if callable(init_weights):
        return init_weights
    if hasattr(top_mod, "_init_weights"):
        return top_mod._init_weights

    def reset(mod):
        if hasattr(mod, "reset_parameters"):
            mod.reset_parameters()

    return reset


def consolidate_model(sch, target=None, init_weights=True, device=None, **kwargs):
    """Materialise and initialise parameters group-consistently (see module doc)."""
    top_mod = sch.mod
    device = torch.device(device) if device is not None else _default_device()
    params = list(top_mod.parameters())
    has_meta = any(p.is_meta for p in params) or any(b.is_meta for b in top_mod.buffers())
    if not init_weights and not has_meta:
        return sch
    if not init_weights and has_meta:
        raise RuntimeError("the model has meta-device parameters; build() needs init_weights")
    init_fn = _pick_init_fn(top_mod, init_weights)
    group = sch.group
    world, rank = sch.world_size, sch.rank
    src_global = dist.get_global_rank(group, 0) if (world > 1 and group is not None) else 0

    done = {}  # old param -> new param (keeps tied weights tied)
    tie = sch.metadata.tie_weights
    mesh = kwargs.get("mesh") if kwargs.get("mesh") is not None else kwargs.get("topology")
    # (a topology object of another kind has no pp_rank: every stage is materialised then)
    my_stage = getattr(mesh, "pp_rank", None) if getattr(mesh, "pp_size", 1) > 1 else None
    visited = set()
    for path, sub in sch.named_schedules():
        mod = sub.mod
        stage = getattr(sub, "partition_idx", None)
        if my_stage is not None and stage is not None and stage != my_stage:
            continue  # another pipeline stage owns this module: leave it unmaterialised
        if id(mod) in visited:
            # one module under several paths (T5's ``shared`` is also ``encoder.embed_tokens``):
            # a second pass would take the fresh parameter for an unknown one, re-create it and
            # so cut it loose from the tensors tied to the first
            continue
        visited.add(id(mod))
        own = [(n, p) for n, p in mod._parameters.items() if p is not None]
        own_bufs = [(n, b) for n, b in mod._buffers.items() if b is not None and b.is_meta]
        if not own and not own_bufs:
            continue
        # 1. full-size stand-ins
        local_shapes, olds = {}, {}
        for n, p in own:
            olds[n] = p
            if p in done:
                continue
            local_shapes[n] = tuple(p.shape)
            full_shape = tuple(getattr(p, "orig_shape", p.shape))
            if p.is_meta:
                full = torch.zeros(full_shape, dtype=p.dtype, device=device)
            elif full_shape != tuple(p.shape):
                # already materialised shard: gather it back so that rank 0's
                # weights win after the broadcast
                axis = _shard_axis(full_shape, p.shape)
                pieces = [torch.empty_like(p.data) for _ in range(world)]
                dist.all_gather(pieces, p.data.contiguous(), group=group)
                full = torch.cat(pieces, dim=axis).to(device)
            else:
                full = p.data.to(device)
            mod._parameters[n] = nn.Parameter(full, requires_grad=p.requires_grad)
        for n, b in own_bufs:
            persistent = n not in mod._non_persistent_buffers_set
            mod.register_buffer(n, torch.zeros(tuple(getattr(b, "orig_shape", b.shape)),
                                               dtype=b.dtype, device=device), persistent)
        # 2. initialise where the module was on meta.  Every rank runs the
        # initialiser (so that all ranks consume the same random numbers and
        # their default RNG streams stay aligned); rank 0's values win below.
        was_meta = any(p.is_meta for _, p in own if p not in done) or bool(own_bufs)
        if was_meta:
            _call_init(init_fn, mod, path)
            _default_init_if_untouched(mod, [n for n, p in own if p.is_meta and p not in done],
                                       init_fn)
        # 3. broadcast + re-split
        for n, old in own:
            if old in done:
                mod._parameters[n] = done[old]
                continue
            full = mod._parameters[n].data
            if world > 1:
                dist.broadcast(full, src=src_global, group=group)
            local_shape = local_shapes[n]
            axis = _shard_axis(tuple(full.shape), local_shape)
            if axis is not None:
                full = full.chunk(world, dim=axis)[rank].contiguous()
            new_param = nn.Parameter(full, requires_grad=old.requires_grad)
            for key, val in vars(old).items():  # orig_shape and user tags
                try:
                    setattr(new_param, key, val)
                except Exception:  # pragma: no cover
                    pass
            transfor_param_tags(sch, old, new_param)
            mod._parameters[n] = new_param
            done[old] = new_param
            for src_param, cur in list(tie.items()):
                if cur is old:
                    tie[src_param] = new_param
    if my_stage is not None:
        # A tensor tied across pipeline stages (word embedding and LM head): the stage modules
        # of other ranks were skipped above and still name the old meta tensor.  They take the
        # new one, so that "the same object in two stages" keeps marking the tie - the pipeline
        # engine finds tied tensors that way, copies the first stage's value to the others and
        # sums their gradients.
        for _, sub in sch.named_schedules():
            for n, old in list(sub.mod._parameters.items()):
                if old is not None and old in done and old is not done[old]:
                    sub.mod._parameters[n] = done[old]
    # tensors that were never on meta (e.g. index buffers) follow to the device
    for mod in top_mod.modules():
        for n, b in list(mod._buffers.items()):
            if b is not None and not b.is_meta and b.device != device:
                mod._buffers[n] = b.to(device)
    if torch.cuda.is_available() and device.type == "cuda":
        torch.cuda.empty_cache()
    return sch


def init_target_engine(sch, target, **kwargs):
    """Hand the scheduled model to the runtime engine of ``target``."""
    engine_cls = get_dialect_cls("runtime_engine", target, allow_none=True)
    return engine_cls(sch, sch.mod, **kwargs)


def build(sch, target=None, init_weights=True, **kwargs):
    """Finish scheduling and return ``(model, optimizer_or_None)``.

    ``init_weights`` is ``True`` (default initialisers), ``False`` (leave
    parameters alone) or a callable ``fn(module)`` / ``fn(module, path)``."""
    from .pipeline import analyze_tie_weights, build_pipeline_model, generate_pipeline_partition

    cuts = sch.metadata.primitives.get("cut_pipeline_stage") or []
    mesh = kwargs.get("mesh") if kwargs.get("mesh") is not None else kwargs.get("topology")
    if not cuts and target is not None and getattr(mesh, "pp_size", 1) > 1:
        raise ValueError(
            f"the mesh has {mesh.pp_size} pipeline stages but the schedule has no "
            "cut_pipeline_stage(): every pipeline rank would train the whole model on its own "
            "(pass pipeline_cuts to the recipe, or build the mesh with pp=1)")
    if cuts:
        sch = generate_pipeline_partition(sch)
        sch.metadata.tie_weights = analyze_tie_weights(sch.mod, is_pipeline_partitioned=True)
    if init_weights:
        sch = consolidate_model(sch, target, init_weights, **kwargs)
    if cuts and target is not None:
        model = build_pipeline_model(sch, target, **kwargs)
        return init_target_engine_for_pipeline(sch, model, target, **kwargs)
    return init_target_engine(sch, target, **kwargs)


def init_target_engine_for_pipeline(sch, model, target, **kwargs):
    engine_cls = get_dialect_cls("runtime_engine", target, allow_none=True)
    return engine_cls(sch, model, **kwargs)
