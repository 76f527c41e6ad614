"""Pipeline partitioning of a traced schedule.

``cut_pipeline_stage`` tags ``call_module`` nodes in the traced graphs of some
ancestors ("a stage ends after this call").  ``generate_pipeline_partition``
turns the tags into stage modules:

1. every traced level between the root and a tagged level is *inlined* into
   the root graph (calls of a GraphModule child are replaced by the child's
   nodes, with dotted module targets, and dict / tuple outputs resolved
   statically), so that all tags end up in one flat graph in program order;
2. the flat graph is split after each tagged node with
   ``torch.fx.passes.split_module`` into ``submod_0 ... submod_{n-1}``;
3. every sub-schedule is stamped with the stage it landed in.

``analyze_pipeline_module`` then computes, for every stage boundary, the
ordered list of values that must cross it: values produced before the boundary
and consumed at or after it (so a tensor needed two stages later is forwarded
through the stage in between).  The runtime exchanges shapes and dtypes of
those lists once and then only moves tensors.

The reference reaches the same stage modules by splitting the lowest traced
level and inlining ``submod_i`` calls upwards level by level
(slapo/pipeline.py:17-183) and encodes the structure of the forwarded tuple in
a metadata tensor that is decoded on the host for every micro-batch
(slapo/framework_dialect/deepspeed/pipeline.py:226-354); here the structure is
static.  Parity for the analysis: slapo/pipeline.py:192-275 and :368-401.
"""
from __future__ import annotations

import operator

from torch import fx
from torch.fx.passes.split_module import split_module

from ..logger import get_logger

logger = get_logger("pipeline")


# ---------------------------------------------------------------------- #
def _resolve_output_access(user: fx.Node, struct):
    """``getitem(out, key)`` / ``out.get(key)`` / ``getattr(out, key)`` on a
    statically known dict / tuple structure -> the selected element."""
    if user.op == "call_function" and user.target is operator.getitem:
        key = user.args[1]
        if isinstance(struct, dict) and isinstance(key, int):
            # a Hugging Face ModelOutput read by position: its fields that are not None, in order
            return [v for v in struct.values() if v is not None][key]
        return struct[key]
    if user.op == "call_method" and user.target == "get":
        return struct.get(user.args[1], user.args[2] if len(user.args) > 2 else None)
    if user.op == "call_function" and user.target is getattr:
        # a field that a traced Hugging Face module left out of its output dict was None
        return struct.get(user.args[1]) if isinstance(struct, dict) else struct[user.args[1]]
    raise RuntimeError(
        f"the output structure of an inlined module is used as a whole by '{user.format_node()}'; "
        "index it (out[...]) in the parent instead")


def inline_call(parent: fx.GraphModule, node: fx.Node):
    """Replace ``node`` (a call of a GraphModule child) by the child's graph."""
    child = parent.get_submodule(node.target)
    if not isinstance(child, fx.GraphModule):
        raise RuntimeError(f"{node.target} is not traced; call trace_until on its path first")
    prefix = node.target
    graph = parent.graph
    placeholders = [n for n in child.graph.nodes if n.op == "placeholder"]
    env = {}
    args = list(node.args)
    for idx, ph in enumerate(placeholders):
        if idx < len(args):
            env[ph] = args[idx]
        elif ph.target in node.kwargs:
            env[ph] = node.kwargs[ph.target]
        elif ph.args:  # default value recorded by fx
            env[ph] = ph.args[0]
        else:
            env[ph] = None
    out_struct = None
    with graph.inserting_before(node):
        for cn in child.graph.nodes:
            if cn.op == "placeholder":
                continue
            if cn.op == "output":
                out_struct = fx.node.map_arg(cn.args[0], lambda n: env[n])
                continue
            new = graph.node_copy(cn, lambda n: env[n])
            if cn.op in ("call_module", "get_attr"):
                new.target = f"{prefix}.{cn.target}"
            new.meta = dict(cn.meta)
            env[cn] = new
    if isinstance(out_struct, fx.Node):
        # a cut on the inlined call itself moves to its last node
        if node.meta.get("partition"):
            out_struct.meta["partition"] = True
        node.replace_all_uses_with(out_struct)
    else:
        for user in list(node.users):
            value = _resolve_output_access(user, out_struct)
            if isinstance(value, fx.Node):
                user.replace_all_uses_with(value)
            else:  # constant (e.g. None): substitute in every use
                for uu in list(user.users):
                    uu.args = fx.node.map_arg(uu.args, lambda n, u=user, v=value: v if n is u else n)
                    uu.kwargs = fx.node.map_arg(uu.kwargs, lambda n, u=user, v=value: v if n is u else n)
            graph.erase_node(user)
        if node.meta.get("partition"):
            last = [n for n in graph.nodes if n.op == "call_module" and n.target.startswith(prefix + ".")]
            if last:
                last[-1].meta["partition"] = True
    graph.erase_node(node)
    graph.lint()
    parent.recompile()


def propagate_partition(sch, cut_paths):
    """Inline every traced level on the way from the root to ``cut_paths``."""
    root = sch.mod
    if not isinstance(root, fx.GraphModule):
        raise RuntimeError("the top module must be traced (trace_until) before cutting stages")
    pending = sorted({p for p in cut_paths if p}, key=lambda p: p.count("."))
    done = set()
    for path in pending:
        tokens = path.split(".")
        for depth in range(1, len(tokens) + 1):
            sub = ".".join(tokens[:depth])
            if sub in done:
                continue
            node = next((n for n in root.graph.nodes if n.op == "call_module" and n.target == sub),
                        None)
            if node is None:
                # ModuleList containers are not called; their elements are
                continue
            inline_call(root, node)
            done.add(sub)
    return root


def generate_pipeline_partition(sch):
    """Split the scheduled model into stage modules ``submod_i`` (see module doc)."""
    cut_paths = sch.metadata.primitives.get("cut_pipeline_stage") or []
    if not cut_paths:
        return sch
    root = propagate_partition(sch, cut_paths)
    stage_of = {}
    stage = 0
    for node in root.graph.nodes:
        stage_of[node] = stage
        if node.op == "call_module" and node.meta.get("partition"):
            stage += 1
    n_stages = stage + 1
    last_compute = [n for n in root.graph.nodes if n.op not in ("placeholder", "output")]
    if last_compute and stage_of[last_compute[-1]] != n_stages - 1:
        n_stages -= 1  # the last cut was on the last node: no empty trailing stage
        for n in stage_of:
            stage_of[n] = min(stage_of[n], n_stages - 1)
    # names under which the unpartitioned model knows its tensors: checkpoints are keyed by
    # them, so that one written by a pipeline loads into any other layout (split_module
    # renames "transformer.h.0" to "transformer_h_0" inside a stage)
    original = {}
    for name, t in list(root.named_parameters(remove_duplicate=False)) \
            + list(root.named_buffers(remove_duplicate=False)):
        original.setdefault(id(t), name)
    split = split_module(root, root, lambda n: stage_of[n], keep_original_order=True)
    for name, sub in split.named_children():
        if name.startswith("submod_"):
            local = list(sub.named_parameters(remove_duplicate=False)) \
                + list(sub.named_buffers(remove_duplicate=False))
            sub.original_tensor_names = {n: original[id(t)] for n, t in local
                                         if id(t) in original}
    # Hooks of the whole model follow what they act on (slapo/pipeline.py:214-226 of the
    # reference): input hooks - a broadcast of the batch inside the tensor-parallel group, say
    # - stay with the top module, and the pipeline engine runs them over the model's inputs
    # where those enter (an encoder-decoder model has inputs that only a later stage reads);
    # backward hooks go to the first stage, output hooks to the last one.
    from ..utils.common import transfer_hooks

    stages = sorted((n for n, _ in split.named_children() if n.startswith("submod_")),
                    key=lambda n: int(n.split("_")[1]))
    transfer_hooks(root, split, ["fwd_pre"])
    if stages:
        transfer_hooks(root, getattr(split, stages[0]), ["bwd_post"])
        transfer_hooks(root, getattr(split, stages[-1]), ["fwd_post"])
    from ..schedule import create_schedule

    new_sch = create_schedule(split, group=sch.group_arg)
    new_sch.metadata.primitives = sch.metadata.primitives
    new_sch.metadata.param_tags = sch.metadata.param_tags
    for name, sub in new_sch.child.items():
        if name.startswith("submod_"):
            idx = int(name.split("_")[1])
            for _, s in sub.named_schedules():
                s.partition_idx = idx
    logger.info("pipeline partition: %d stages", n_stages, ranks=0)
    return new_sch


# ---------------------------------------------------------------------- #
def analyze_pipeline_module(top_mod: fx.GraphModule):
    """Data contract between the stages of a split module.

    Returns ``(stage_inputs, stage_names, live_in)``:

    * ``stage_names[i]``  - attribute name of stage i (``submod_i``);
    * ``stage_inputs[i]`` - names of the values stage i's module takes, in its
      argument order;
    * ``live_in[i]``      - ordered names of the values that cross the boundary
      into stage i (``live_in[0]`` are the model inputs).  ``live_in[i + 1]`` is
      what stage i must send on, including values it only forwards.
    """
    graph = top_mod.graph
    calls = [n for n in graph.nodes if n.op == "call_module" and n.target.startswith("submod_")]
    stage_of_value = {}
    names = {}
    for n in graph.nodes:
        names[n] = n.name
    for n in graph.nodes:
        if n.op == "placeholder":
            stage_of_value[n] = -1
    for i, call in enumerate(calls):
        stage_of_value[call] = i
    # getitem on a stage result belongs to that stage
    for n in graph.nodes:
        if n.op == "call_function" and n.target is operator.getitem and n.args[0] in stage_of_value:
            stage_of_value[n] = stage_of_value[n.args[0]]
    stage_inputs, stage_names = [], []
    last_use = {}
    n_stages = len(calls)
    for i, call in enumerate(calls):
        stage_names.append(call.target)
        stage_inputs.append([names[a] for a in call.all_input_nodes])
        for a in call.all_input_nodes:
            last_use[a] = i
    out_node = next(n for n in graph.nodes if n.op == "output")
    for a in out_node.all_input_nodes:
        last_use[a] = n_stages  # the final result leaves the last stage
    live_in = []
    for i in range(n_stages):
        live = [names[v] for v, s in stage_of_value.items()
                if s < i and last_use.get(v, -1) >= i and not (
                    v.op == "call_module" and any(
                        u.op == "call_function" and u.target is operator.getitem for u in v.users))]
        live_in.append(live)
    return stage_inputs, stage_names, live_in


def stage_output_names(top_mod: fx.GraphModule):
    """For every stage: ``[(value_name, index_or_None), ...]`` - how the return
    value of the stage module maps to the value names used by ``live_in``."""
    calls = [n for n in top_mod.graph.nodes
             if n.op == "call_module" and n.target.startswith("submod_")]
    out = []
    for call in calls:
        items = [(u.name, u.args[1]) for u in call.users
                 if u.op == "call_function" and u.target is operator.getitem]
        out.append(items if items else [(call.name, None)])
    return out


def final_output_spec(top_mod: fx.GraphModule):
    """The structure returned by the whole model, with value names as leaves."""
    out_node = next(n for n in top_mod.graph.nodes if n.op == "output")
    return fx.node.map_arg(out_node.args[0], lambda n: n.name)


def build_pipeline_model(sch, target, **kwargs):
    """Wrap the stage modules for ``target`` and assemble the pipeline model."""
    from ..framework_dialect import get_dialect_cls

    stage_inputs, stage_names, live_in = analyze_pipeline_module(sch.mod)
    stage_cls = get_dialect_cls("pipeline_stage", target)
    engine_cls = get_dialect_cls("pipeline_engine", target)
    stages = []
    top_attrs = {}
    for node in sch.mod.graph.nodes:
        if node.op == "get_attr":
            value = sch.mod
            for tok in node.target.split("."):
                value = getattr(value, tok)
            top_attrs[node.name] = value
    for i, name in enumerate(stage_names):
        consts = {n: top_attrs[n] for n in stage_inputs[i] if n in top_attrs}
        extra = {"constants": consts} if consts else {}
        stages.append(stage_cls(getattr(sch.mod, name), i, len(stage_names), stage_inputs[i],
                                stage_output_names(sch.mod)[i], **extra))
    input_names = [n.name for n in sch.mod.graph.nodes if n.op == "placeholder"]
    return engine_cls(stages, live_in=live_in, input_names=input_names,
                      output_spec=final_output_spec(sch.mod),
                      input_hooks=list(sch.mod._forward_pre_hooks.values()))
