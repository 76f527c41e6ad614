"""``replace`` and ``replace_all``.

``sch.replace(new, target_ops=None, name=None, concrete_args=None)`` has three
forms:

* ``target_ops is None`` - swap the whole module of this schedule node by the
  module ``new``; hooks move over, a fresh sub-schedule tree is created and
  the parent module (attribute or ModuleList slot) is updated;
* ``target_ops`` is a list of sub-graphs from ``find`` - one sub-graph is a
  *vertical* replacement (the chain becomes one call of ``new`` placed after
  its last node), several sub-graphs are a *horizontal* replacement (the N
  parallel branches become one call whose i-th output feeds branch i's users);
* ``target_ops`` is a single ``(parent_name, node)`` pair and ``new`` is a
  function - retarget that ``call_function`` node.

``sch.replace_all(cls, make_mod_fn, **kw)`` swaps every module of type ``cls``
below this node by ``make_mod_fn(name, module, **kw)``.

Parity: slapo/primitives/replace.py:21-389 of the reference.  One deliberate
difference: default-valued parameters of the new module are handled
correctly (the reference iterates the dictionary of defaults by key and
raises for any module with defaults).
"""
from __future__ import annotations

import inspect
import operator
from types import BuiltinFunctionType, FunctionType

from torch import fx, nn

from ..logger import get_logger
from ..utils.common import transfer_hooks, transfer_hooks_for_fusion
from .base import Primitive, register_primitive

logger = get_logger("replace")


def _get_unique_module_name(gm_or_modules, name: str) -> str:
    """First free ``name_k`` (k = 0, 1, ...) among the module names."""
    if isinstance(gm_or_modules, nn.Module):
        taken = set(dict(gm_or_modules.named_modules()).keys())
    else:
        taken = set(gm_or_modules)
    k = 0
    while f"{name}_{k}" in taken:
        k += 1
    return f"{name}_{k}"


def _is_function(obj) -> bool:
    return isinstance(obj, (FunctionType, BuiltinFunctionType)) or (
        callable(obj) and not isinstance(obj, nn.Module))


def _external_inputs(ops):
    """Values read by the chain that it does not produce, in first-use order."""
    inside = set(ops)
    seen, out = set(), []
    for node in ops:
        for inp in node.all_input_nodes:
            if inp not in inside and inp not in seen:
                seen.add(inp)
                out.append(inp)
    return out


def _check_arity(new_mod_or_func, n_inputs: int, concrete_args):
    target = new_mod_or_func.forward if isinstance(new_mod_or_func, nn.Module) else new_mod_or_func
    try:
        sig = inspect.signature(target)
    except (ValueError, TypeError):
        return
    params = list(sig.parameters.values())
    if any(p.kind is p.VAR_POSITIONAL for p in params):
        return
    concrete = set((concrete_args or {}).keys())
    required = [p for p in params if p.default is inspect.Parameter.empty
                and p.kind is not p.VAR_KEYWORD and p.name not in concrete]
    positional = [p for p in params if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)
                  and p.name not in concrete]
    if n_inputs < len(required) or n_inputs > len(positional):
        raise ValueError(
            f"the replacement takes {len(required)} required argument(s) "
            f"(at most {len(positional)}), but the matched sub-graph has {n_inputs} "
            "external input(s); use `concrete_args` to bind the extra ones")


def _owner_module(root: nn.Module, path: str) -> nn.Module:
    if not path:
        return root
    owner = dict(root.named_modules()).get(path)
    if owner is None:
        raise RuntimeError(f"'{path}' is not a sub-module of {type(root).__name__}")
    return owner


def _last_in_program_order(graph: fx.Graph, nodes):
    pos = {n: i for i, n in enumerate(graph.nodes)}
    return max(nodes, key=lambda n: pos[n])


def _insert_call(owner, graph, after, new_mod_or_func, name, args, kwargs):
    with graph.inserting_after(after):
        if isinstance(new_mod_or_func, nn.Module):
            return graph.call_module(name, tuple(args), dict(kwargs))
        return graph.call_function(new_mod_or_func, tuple(args), dict(kwargs))


def _erase_chain(graph, ops):
    pos = {n: i for i, n in enumerate(graph.nodes)}
    for node in sorted(ops, key=lambda n: -pos[n]):
        if len(node.users) == 0:
            graph.erase_node(node)


def _subgraph_replace(sch, new_mod_or_func, subgraphs, name, concrete_args):
    """Vertical (1 sub-graph) or horizontal (>1) replacement."""
    path = subgraphs[0][0][0]
    if any(p != path for sub in subgraphs for p, _ in sub):
        raise ValueError("all matched nodes must live in the same traced module")
    owner = _owner_module(sch.mod, path)
    if not isinstance(owner, fx.GraphModule):
        raise RuntimeError("sub-graph replacement needs a traced module")
    graph = owner.graph
    chains = [[node for _, node in sub] for sub in subgraphs]
    is_module = isinstance(new_mod_or_func, nn.Module)

    if is_module:
        if name is None:
            name = type(new_mod_or_func).__name__
        name = _get_unique_module_name(owner, name)
        new_mod_or_func.train(owner.training)
        owner.add_module(name, new_mod_or_func)

    if len(chains) == 1:
        ops = chains[0]
        inputs = _external_inputs(ops)
        _check_arity(new_mod_or_func, len(inputs), concrete_args)
        last = _last_in_program_order(graph, ops)
        new_node = _insert_call(owner, graph, last, new_mod_or_func, name, inputs,
                                concrete_args or {})
        last.replace_all_uses_with(new_node, delete_user_cb=lambda u: u is not new_node)
        _erase_chain(graph, ops)
    else:
        # every branch must read the same external inputs
        inputs = _external_inputs(chains[0])
        for ops in chains[1:]:
            if _external_inputs(ops) != inputs:
                raise ValueError("horizontal replacement needs branches with identical inputs")
        _check_arity(new_mod_or_func, len(inputs), concrete_args)
        lasts = [_last_in_program_order(graph, ops) for ops in chains]
        # place the fused call where the first branch ends; its inputs are
        # defined before every branch, and every user comes after that point
        # only if it follows all branch heads, so hoist the call to just
        # after the latest input definition instead
        pos = {n: i for i, n in enumerate(graph.nodes)}
        anchor = max(inputs, key=lambda n: pos[n]) if inputs else next(iter(graph.nodes))
        new_node = _insert_call(owner, graph, anchor, new_mod_or_func, name, inputs,
                                concrete_args or {})
        prev = new_node
        for idx, last in enumerate(lasts):
            with graph.inserting_after(prev):
                item = graph.call_function(operator.getitem, (new_node, idx))
            last.replace_all_uses_with(item)
            prev = item
        for ops in chains:
            _erase_chain(graph, ops)

    if is_module:
        transfer_hooks_for_fusion(sch, subgraphs, new_mod_or_func)
    _finalize_graph(owner)
    return name


def _finalize_graph(gm: fx.GraphModule):
    gm.graph.eliminate_dead_code()
    gm.delete_all_unused_submodules()
    gm.graph.lint()
    gm.recompile()


def _function_replace(sch, new_func, target_op):
    path, node = target_op
    owner = _owner_module(sch.mod, path)
    if node.op != "call_function":
        raise ValueError("function replacement needs a call_function node")
    with owner.graph.inserting_after(node):
        new_node = owner.graph.call_function(new_func, node.args, node.kwargs)
    node.replace_all_uses_with(new_node)
    owner.graph.erase_node(node)
    _finalize_graph(owner)


def _module_replace(sch, new_mod: nn.Module):
    from ..schedule import create_schedule

    if new_mod is sch.mod:
        return
    transfer_hooks(sch.mod, new_mod)
    new_mod.train(sch.mod.training)  # a fresh module defaults to training mode
    new_sch = create_schedule(new_mod, sch.name, sch.path, sch.parent, sch.group_arg)
    sch.mod = new_mod
    sch.child = new_sch.child
    for child in sch.child.values():
        child.parent = sch
    if sch.parent is not None:
        sch.update_submodule(sch.parent.mod, sch.name, new_mod)


def _resync_children(sch):
    """After a graph edit: drop schedules of deleted sub-modules, add
    schedules for new ones, keep the untouched ones (they carry metadata)."""
    from ..schedule import create_schedule

    fresh = create_schedule(sch.mod, sch.name, sch.path, sch.parent, sch.group_arg)
    merged = {}
    for key, child in fresh.child.items():
        old = sch.child.get(key)
        if old is not None and old.mod is child.mod:
            merged[key] = old
        else:
            child.parent = sch
            merged[key] = child
    sch.child = merged


@register_primitive()
class ReplacePrimitive(Primitive):
    @staticmethod
    def name():
        return "replace"

    @staticmethod
    def apply(sch, new_mod_or_func, target_ops=None, name=None, concrete_args=None):
        if target_ops is None:
            if not isinstance(new_mod_or_func, nn.Module):
                raise ValueError("whole-module replacement needs an nn.Module")
            _module_replace(sch, new_mod_or_func)
            return None
        if isinstance(target_ops, tuple) and len(target_ops) == 2 and isinstance(target_ops[1], fx.Node):
            target_ops = [[target_ops]] if isinstance(new_mod_or_func, nn.Module) else target_ops
        if isinstance(target_ops, tuple):
            if not _is_function(new_mod_or_func):
                raise ValueError("a single-node target needs a function replacement")
            _function_replace(sch, new_mod_or_func, target_ops)
            _resync_children(sch)
            return None
        if not target_ops:
            raise ValueError("target_ops is empty: nothing matched")
        if isinstance(target_ops[0], tuple):  # one flat chain
            target_ops = [target_ops]
        if name is None and not isinstance(new_mod_or_func, nn.Module):
            name = getattr(new_mod_or_func, "__name__", "func")
        new_name = _subgraph_replace(sch, new_mod_or_func, target_ops, name, concrete_args)
        _resync_children(sch)
        return new_name


@register_primitive()
class ReplaceAllPrimitive(Primitive):
    @staticmethod
    def name():
        return "replace_all"

    @staticmethod
    def apply(sch, target_mod_type, make_mod_fn, **kwargs):
        # snapshot first: replacements must not be descended into
        victims = [(n, s) for n, s in sch.named_schedules() if isinstance(s.mod, target_mod_type)]
        for sub_name, sub_sch in victims:
            new_mod = make_mod_fn(sub_name, sub_sch.mod, **kwargs)
            if new_mod is not None:
                sub_sch.replace(new_mod)
        return len(victims)
