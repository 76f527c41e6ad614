"""Implementation of the sharded checkpoint format described in the package
docstring."""
from __future__ import annotations

import json
import os
import random as _py_random
import re

import numpy as np
import torch
import torch.distributed as dist

from ..logger import get_logger
from ..random import get_cuda_rng_tracker

logger = get_logger("ckpt")

FORMAT_VERSION = 1
_STATE_KEYS = ("master", "exp_avg", "exp_avg_sq")
_STAGE_PREFIX = re.compile(r"^(?:stages?\.\d+\.|submod_\d+\.)+")


def canonical_name(name: str) -> str:
    """Parameter name without pipeline-stage wrappers (``submod_3.``,
    ``stage.2.``), so that checkpoints of different pipeline layouts agree."""
    return _STAGE_PREFIX.sub("", name)


def _coords(mesh, model=None):
    """This rank's (pp, dp, tp) coordinates, the mesh dimensions and the global rank.

    Without a mesh a job of several ranks is read as ONE tensor-parallel group over the whole
    world when the model carries sharded tensors (``create_schedule(model)`` with the default
    group shards over all ranks), and as plain data parallelism when it does not - so that
    the ranks never write the same shard file with different contents."""
    if mesh is not None:
        coord = mesh.get_coord()
        return dict(coord), dict(mesh.dims), mesh.rank
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return {"pp": 0, "dp": 0, "tp": 0}, {"pp": 1, "dp": 1, "tp": 1}, 0
    rank, world = dist.get_rank(), dist.get_world_size()
    sharded = model is not None and any(
        tuple(getattr(t, "orig_shape", t.shape)) != tuple(t.shape)
        for _, t in _unique_named_tensors(model))
    # every rank must take the same branch: a rank whose own tensors happen to be whole still
    # belongs to the tensor-parallel group of its peers
    flag = torch.tensor([1 if sharded else 0])
    if dist.get_backend() == "nccl":
        flag = flag.cuda()
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if int(flag.item()):
        return {"pp": 0, "dp": 0, "tp": rank}, {"pp": 1, "dp": 1, "tp": world}, rank
    return {"pp": 0, "dp": rank, "tp": 0}, {"pp": 1, "dp": world, "tp": 1}, rank


def _shard_axis(full_shape, local_shape):
    diff = [i for i, (a, b) in enumerate(zip(full_shape, local_shape)) if a != b]
    if len(diff) > 1:
        raise RuntimeError(f"more than one sharded axis: {full_shape} -> {local_shape}")
    return diff[0] if diff else None


def original_names(model):
    """``{name inside model: name in the unpartitioned model}`` for the tensors of pipeline
    stage modules (the partitioner records them as ``original_tensor_names``); empty for a
    model that was never partitioned."""
    out = {}
    for prefix, mod in model.named_modules():
        table = getattr(mod, "original_tensor_names", None)
        if isinstance(table, dict):
            for local, orig in table.items():
                out[f"{prefix}.{local}" if prefix else local] = orig
    return out


def _namer(model):
    table = original_names(model)
    return lambda name: table[name] if name in table else canonical_name(name)


def _tensor_groups(model):
    """``[(names, tensor)]`` for parameters and persistent buffers: ``names`` are all the
    (canonical) names under which the model holds the tensor - a tied tensor has several -
    and the first one is the name it is stored under."""
    namer = _namer(model)
    skip = set()
    for mod_name, mod in model.named_modules():
        for b in getattr(mod, "_non_persistent_buffers_set", ()):
            skip.add(f"{mod_name}.{b}" if mod_name else b)
    groups, index = [], {}
    named = list(model.named_parameters(remove_duplicate=False)) + [
        (n, b) for n, b in model.named_buffers(remove_duplicate=False) if n not in skip]
    for name, t in named:
        canon = namer(name)
        if id(t) in index:
            names = groups[index[id(t)]][0]
            if canon not in names:
                names.append(canon)
            continue
        index[id(t)] = len(groups)
        groups.append(([canon], t))
    return groups


def _unique_named_tensors(model):
    """(canonical name, tensor) for parameters and persistent buffers; a tied
    parameter appears once, under its first name."""
    for names, t in _tensor_groups(model):
        yield names[0], t


def _rng_state():
    state = {"python": _py_random.getstate(), "numpy": np.random.get_state(),
             "torch": torch.get_rng_state(), "tracker": get_cuda_rng_tracker().get_states()}
    if torch.cuda.is_available():
        state["cuda"] = torch.cuda.get_rng_state()
    return state


def _set_rng_state(state):
    _py_random.setstate(state["python"])
    np.random.set_state(state["numpy"])
    torch.set_rng_state(state["torch"])
    if "cuda" in state and torch.cuda.is_available():
        torch.cuda.set_rng_state(state["cuda"])
    get_cuda_rng_tracker().set_states(state["tracker"])


def _barrier():
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


# ---------------------------------------------------------------------- #
def _unwrap(model, engine):
    """A pipeline engine stands for its stage: the engine that owns this rank's parameters is
    ``engine.inner`` and the module to save or fill is that engine's stage module (the other
    stages of the pipeline model live on other ranks)."""
    inner = getattr(engine, "inner", None)
    if inner is not None and hasattr(inner, "full_optimizer_state"):
        if model is None or model is getattr(engine, "model", None):
            model = inner.model
        engine = inner
    if model is None and engine is not None:
        model = engine.model
    return model, engine


def save_checkpoint(path, model, engine=None, mesh=None, step=None, extra=None):
    """Write this rank's part of a checkpoint into directory ``path``.
    Collective: every rank of the job calls it.  ``engine`` may be a pipeline engine (then
    ``model`` may be its pipeline model, or None)."""
    model, engine = _unwrap(model, engine)
    if mesh is None:
        mesh = getattr(engine, "mesh", None)
    coord, dims, rank = _coords(mesh, model)
    os.makedirs(path, exist_ok=True)
    tag = f"pp{coord['pp']}_tp{coord['tp']}"
    table, tensors = {}, {}
    for names, t in _tensor_groups(model):
        name = names[0]
        full_shape = tuple(getattr(t, "orig_shape", t.shape))
        table[name] = {"shape": list(t.shape), "orig_shape": list(full_shape),
                       "axis": _shard_axis(full_shape, tuple(t.shape)),
                       "dtype": str(t.dtype).replace("torch.", ""), "stage": coord["pp"]}
        if len(names) > 1:
            # other names of a tied tensor: a model in another layout may know it by one of
            # them only (a pipeline stage holds "lm_head.weight" but not "wte.weight")
            table[name]["aliases"] = names[1:]
        tensors[name] = t.detach().cpu()
    # optimizer state is gathered over DP by every rank (collective), written by DP rank 0
    optim = None
    if engine is not None:
        optim = engine.full_optimizer_state(to_cpu=True)
        namer = _namer(model)
        optim["state"] = {namer(k): v for k, v in optim["state"].items()}
        if step is None:
            step = optim["step"]
    if coord["dp"] == 0:
        torch.save(tensors, os.path.join(path, f"model_{tag}.pt"))
        if optim is not None:
            torch.save(optim, os.path.join(path, f"optim_{tag}.pt"))
        with open(os.path.join(path, f"table_{tag}.json"), "w", encoding="utf-8") as fh:
            json.dump(table, fh)
    torch.save(_rng_state(), os.path.join(path, f"rng_rank{rank}.pt"))
    _barrier()
    if rank == 0:
        params = {}
        for pp in range(dims["pp"]):
            # the table of TP rank 0 of each stage describes the stage
            with open(os.path.join(path, f"table_pp{pp}_tp0.json"), encoding="utf-8") as fh:
                params.update(json.load(fh))
        manifest = {"version": FORMAT_VERSION, "step": int(step or 0), "mesh": dims,
                    "has_optimizer": engine is not None, "params": params}
        with open(os.path.join(path, "manifest.json"), "w", encoding="utf-8") as fh:
            json.dump(manifest, fh, indent=1)
        if extra is not None:
            torch.save(extra, os.path.join(path, "extra.pt"))
        logger.info("saved checkpoint step %d to %s (%d tensors/stage-0 shard)", manifest["step"],
                    path, len(tensors))
    _barrier()
    return path


def read_manifest(path):
    with open(os.path.join(path, "manifest.json"), encoding="utf-8") as fh:
        manifest = json.load(fh)
    if manifest.get("version") != FORMAT_VERSION:
        raise ValueError(f"unsupported checkpoint version {manifest.get('version')}")
    return manifest


def _load_file(path, name):
    return torch.load(os.path.join(path, name), map_location="cpu", weights_only=False)


def _merge_tp(pieces, axis, name=None, full_shape=None):
    out = pieces[0] if axis is None else torch.cat(pieces, dim=axis)
    if full_shape is not None and tuple(out.shape) != tuple(full_shape):
        raise ValueError(f"{name}: the shards put together have shape {tuple(out.shape)}, the "
                         f"manifest records {tuple(full_shape)}: the checkpoint's shard files "
                         "do not belong to one tensor-parallel layout")
    return out


def consolidate_checkpoint(path, with_optimizer=False, out_file=None):
    """Full (unsharded) tensors of a checkpoint: ``{name: tensor}``, or
    ``(weights, {"step", "state": {name: {...}}})`` with the optimizer."""
    manifest = read_manifest(path)
    dims, table = manifest["mesh"], manifest["params"]
    weights, optim = {}, {"step": manifest["step"], "state": {}}
    for pp in range(dims["pp"]):
        shards = [_load_file(path, f"model_pp{pp}_tp{tp}.pt") for tp in range(dims["tp"])]
        for name in shards[0]:
            weights[name] = _merge_tp([s[name] for s in shards], table[name]["axis"], name,
                                      table[name]["orig_shape"])
        if with_optimizer and manifest["has_optimizer"]:
            opt = [_load_file(path, f"optim_pp{pp}_tp{tp}.pt") for tp in range(dims["tp"])]
            optim["step"] = opt[0]["step"]
            for name in opt[0]["state"]:
                optim["state"][name] = {
                    key: _merge_tp([o["state"][name][key] for o in opt], table[name]["axis"])
                    for key in _STATE_KEYS}
    if out_file is not None:
        torch.save(weights, out_file)
    return (weights, optim) if with_optimizer else weights


def _slice_for(full, local_shape, axis_hint, tp_rank, tp_size, name):
    if tuple(full.shape) == tuple(local_shape):
        return full
    axis = _shard_axis(tuple(full.shape), tuple(local_shape))
    if axis is None or full.shape[axis] != local_shape[axis] * tp_size:
        raise ValueError(f"{name}: checkpoint tensor {tuple(full.shape)} cannot be split into "
                         f"{tp_size} shards of {tuple(local_shape)}")
    if axis_hint is not None and axis_hint != axis:
        logger.warning("%s was saved sharded along axis %d, now along %d", name, axis_hint, axis)
    return full.chunk(tp_size, dim=axis)[tp_rank]


def load_checkpoint(path, model, engine=None, mesh=None, strict=True, load_rng=True):
    """Load weights (and, with ``engine``, optimizer state) into this rank's
    model.  The checkpoint may have been written with another DP size, ZeRO
    setting or TP size: tensors whose saved shard shape differs from the
    model's are consolidated along their recorded axis and re-split.
    ``engine`` may be a pipeline engine.  Returns ``{"step", "extra"}``."""
    manifest = read_manifest(path)
    model, engine = _unwrap(model, engine)
    if mesh is None:
        mesh = getattr(engine, "mesh", None)
    coord, dims, rank = _coords(mesh, model)
    saved = manifest["mesh"]
    table = manifest["params"]
    same_layout = saved["tp"] == dims["tp"] and saved["pp"] == dims["pp"]
    if same_layout:
        tag = f"pp{coord['pp']}_tp{coord['tp']}"
        weights = _load_file(path, f"model_{tag}.pt")
        optim = _load_file(path, f"optim_{tag}.pt") if (
            engine is not None and manifest["has_optimizer"]) else None
    else:
        need_opt = engine is not None and manifest["has_optimizer"]
        result = consolidate_checkpoint(path, with_optimizer=need_opt)
        weights, optim = result if need_opt else (result, None)
    missing, loaded = [], set()
    alias_of = {a: primary for primary, e in table.items() for a in e.get("aliases", ())}

    def stored_name(names, pool):
        """The name under which the checkpoint holds the tensor this model calls ``names``."""
        for n in names:
            if n in pool:
                return n
            if alias_of.get(n) in pool:
                return alias_of[n]
        return None

    with torch.no_grad():
        for names, t in _tensor_groups(model):
            name = stored_name(names, weights)
            if name is None:
                missing.append(names[0])
                continue
            hint = table.get(name, {}).get("axis")
            src = _slice_for(weights[name], t.shape, hint, coord["tp"], dims["tp"], name)
            t.copy_(src.to(t.dtype))
            loaded.add(name)
    unexpected = [] if not same_layout and dims["pp"] > 1 else [n for n in weights if n not in loaded]
    if strict and (missing or unexpected):
        raise KeyError(f"checkpoint mismatch: missing {missing[:5]}, unexpected {unexpected[:5]}")
    if engine is not None:
        if optim is not None:
            local = {"step": optim["step"], "state": {}}
            namer = _namer(model)
            groups = {names[0]: names for names, _ in _tensor_groups(model)}
            params = dict(model.named_parameters())
            for local_name in engine._param_names():
                names = groups.get(namer(local_name), [namer(local_name)])
                name = stored_name(names, optim["state"])
                if name is None:
                    continue
                entry, shape = optim["state"][name], params[local_name].shape
                hint = table.get(name, {}).get("axis")
                local["state"][local_name] = {
                    key: _slice_for(entry[key], shape, hint, coord["tp"], dims["tp"], name)
                    for key in _STATE_KEYS}
            engine.load_full_optimizer_state(local)
        else:
            engine.refresh_master_from_params()
    rng_file = os.path.join(path, f"rng_rank{rank}.pt")
    if load_rng and same_layout and saved["dp"] == dims["dp"] and os.path.exists(rng_file):
        _set_rng_state(torch.load(rng_file, map_location="cpu", weights_only=False))
    extra = None
    if os.path.exists(os.path.join(path, "extra.pt")):
        extra = _load_file(path, "extra.pt")
    _barrier()
    return {"step": manifest["step"], "extra": extra}


def reshard_checkpoint(src, dst, tp_size, stage_of=None, pp_size=1):
    """Rewrite checkpoint ``src`` for ``tp_size`` tensor-parallel ranks (and,
    with ``stage_of(name) -> stage``, ``pp_size`` pipeline stages) into ``dst``.
    Runs on one process, no GPU needed.  Every tensor that was sharded stays
    sharded along the same axis; replicated tensors stay replicated."""
    manifest = read_manifest(src)
    table = manifest["params"]
    has_opt = manifest["has_optimizer"]
    result = consolidate_checkpoint(src, with_optimizer=has_opt)
    weights, optim = result if has_opt else (result, None)
    os.makedirs(dst, exist_ok=True)
    new_table = {}
    for pp in range(pp_size):
        names = [n for n in weights if (stage_of(n) if stage_of else 0) == pp]
        for tp in range(tp_size):
            shard, opt_shard = {}, {"step": manifest["step"], "state": {}}
            for name in names:
                axis = table[name]["axis"]
                full = weights[name]
                if axis is not None and full.shape[axis] % tp_size:
                    raise ValueError(f"{name}: axis {axis} of {tuple(full.shape)} is not divisible "
                                     f"by {tp_size}")
                cut = (lambda t, a=axis: t if a is None else t.chunk(tp_size, dim=a)[tp].clone())
                shard[name] = cut(full)
                if optim is not None and name in optim["state"]:
                    opt_shard["state"][name] = {k: cut(optim["state"][name][k]) for k in _STATE_KEYS}
                if tp == 0:
                    new_table[name] = dict(table[name], shape=list(shard[name].shape), stage=pp)
            torch.save(shard, os.path.join(dst, f"model_pp{pp}_tp{tp}.pt"))
            if optim is not None:
                opt_shard["step"] = optim["step"]
                torch.save(opt_shard, os.path.join(dst, f"optim_pp{pp}_tp{tp}.pt"))
    new_manifest = dict(manifest, mesh={"pp": pp_size, "dp": 1, "tp": tp_size}, params=new_table)
    with open(os.path.join(dst, "manifest.json"), "w", encoding="utf-8") as fh:
        json.dump(new_manifest, fh, indent=1)
    if os.path.exists(os.path.join(src, "extra.pt")):
        torch.save(_load_file(src, "extra.pt"), os.path.join(dst, "extra.pt"))
    return dst
