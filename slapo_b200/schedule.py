"""The schedule tree.

``create_schedule(model)`` mirrors an ``nn.Module`` hierarchy with a tree of
``Schedule`` nodes.  Each node exposes every registered primitive as a bound
method (``sch["encoder.layer.0.attention"].shard("weight", 0)``) plus the
static-graph queries ``trace`` / ``trace_until`` / ``find`` / ``find_node`` /
``find_subgraph``.

Tree rules (parity: slapo/schedule.py:509-581 of the reference):

* a module from ``torch.nn`` that is not an ``nn.Sequential`` is a leaf (the bare containers
  of a flattened trace included; those a hierarchical trace leaves above a grandchild call
  are not);
* the elements of a ``ModuleList`` become children named ``"<list>.<i>"``
  (one path token); everything else, ``nn.Sequential`` included, is a direct
  child, so ``sch["seq"]["0"]`` and ``sch["seq.0"]`` both work.
"""
from __future__ import annotations

import re
from types import FunctionType
from typing import Callable, Optional

import torch.distributed as dist
from torch import fx, nn

from .graph.matcher import SubgraphMatcher
from .graph.tracer import trace as trace_module
from .logger import get_logger
from .pattern import Pattern
from .primitives.base import PRIMITIVES
from .utils.common import is_module_list

logger = get_logger("schedule")


class ScheduleMetadata:
    """State shared along a schedule tree.

    ``tie_weights`` maps each originally shared Parameter to its current
    replacement (one dict for the whole tree), ``param_tags`` is the set of
    attribute names that must follow a parameter when it is re-created, and
    ``primitives`` holds per-primitive notes (e.g. the shard axis per tensor).
    """

    def __init__(self):
        self.tie_weights = {}
        self.param_tags = set()
        self.primitives = {}


class Schedule:
    def __init__(self, mod: nn.Module, name: str = "", path: str = "",
                 parent: Optional["Schedule"] = None, group=None):
        # what to hand to create_schedule() to get a schedule over the same ranks again
        # (``group`` itself becomes None for the "no tensor parallelism" sentinel)
        self.group_arg = group
        if group is False:  # explicit "no tensor parallelism" inside a distributed job
            self.world_size, self.rank, group = 1, 0, None
        elif dist.is_available() and dist.is_initialized():
            self.world_size = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
        else:
            self.world_size, self.rank = 1, 0
        self.group = group
        self.mod = mod
        self.name = name
        self.path = path
        self.parent = parent
        self.child: dict[str, Schedule] = {}
        self.metadata = ScheduleMetadata()
        if parent is None:
            from .pipeline import analyze_tie_weights

            for param in analyze_tie_weights(mod, False):
                self.metadata.tie_weights[param] = param
        else:
            self.metadata.tie_weights = parent.metadata.tie_weights
            self.metadata.param_tags = parent.get_top_schedule().metadata.param_tags
        for pname, cls in PRIMITIVES.items():
            self.metadata.primitives[pname] = cls.init_metadata()

    # primitives are looked up lazily so that primitives registered after the
    # schedule was created are available too
    def __getattr__(self, item):
        prims = PRIMITIVES
        if item in prims:
            cls = prims[item]

            def bound(*args, **kwargs):
                return cls.apply(self, *args, **kwargs)

            bound.__name__ = item
            bound.__doc__ = cls.apply.__doc__
            return bound
        raise AttributeError(f"'Schedule' object has no attribute or primitive '{item}'")

    def __repr__(self):
        return f"Schedule(path='{self.path}', mod={type(self.mod).__name__}, children={list(self.child)})"

    # ------------------------------------------------------------------ #
    # path handling
    @staticmethod
    def tokenize_module_path(module_path: str) -> list[str]:
        """``"a.b.0.c"`` -> ``["a", "b.0", "c"]`` (an index joins its list; a
        leading index, as in ``sch["layer1"]["0"]``, names a child of an
        ``nn.Sequential`` and stays a token of its own)."""
        tokens: list[str] = []
        for piece in module_path.split("."):
            if piece.isdigit():
                if not tokens:
                    tokens.append(piece)
                    continue
                tokens[-1] = f"{tokens[-1]}.{piece}"
            else:
                tokens.append(piece)
        return tokens

    @staticmethod
    def update_submodule(mod: nn.Module, submod_name: str, new_submod: nn.Module):
        if "." in submod_name:
            list_name, idx = submod_name.split(".")
            container = getattr(mod, list_name)
            if isinstance(container, (nn.ModuleList, nn.Sequential)):
                container[int(idx)] = new_submod
            else:
                setattr(container, idx, new_submod)
        else:
            setattr(mod, submod_name, new_submod)

    def _walk(self, full_path):
        cur = self
        for token in self.tokenize_module_path(full_path):
            if token not in cur.child:
                head, _, tail = token.partition(".")
                if tail and head in cur.child and tail in cur.child[head].child:
                    cur = cur.child[head].child[tail]  # "seq.0" through nn.Sequential
                    continue
                return None, token, cur
            cur = cur.child[token]
        return cur, None, None

    def __getitem__(self, full_path: str) -> "Schedule":
        if not full_path:
            return self
        found, token, where = self._walk(full_path)
        if found is None:
            raise KeyError(
                f"'{full_path}': '{token}' is not a child of schedule '{where.path or '<root>'}' "
                f"(children: {list(where.child)})")
        return found

    def __contains__(self, full_path: str) -> bool:
        if not full_path:
            return True
        try:
            return self._walk(full_path)[0] is not None
        except KeyError:
            return False

    def get_top_schedule(self) -> "Schedule":
        cur = self
        while cur.parent is not None:
            cur = cur.parent
        return cur

    def get_module(self, name: str) -> nn.Module:
        return dict(self.mod.named_modules())[name]

    def named_schedules(self, prefix: str = ""):
        yield prefix, self
        for name, sub in self.child.items():
            yield from sub.named_schedules(f"{prefix}.{name}" if prefix else name)

    # ------------------------------------------------------------------ #
    # static graph
    def trace(self, **kwargs) -> bool:
        """Replace ``self.mod`` by its traced GraphModule tree.

        No-op when already traced.  Returns False (with a warning) when the
        module cannot be traced."""
        if isinstance(self.mod, fx.GraphModule):
            return True
        failed_msg = None
        try:
            gm = trace_module(self.mod, **kwargs)
        except Exception as err:  # pragma: no cover - trace() itself degrades
            gm, failed_msg = self.mod, str(err)
        if not isinstance(gm, fx.GraphModule):
            logger.warning("failed to trace %s %s", self.path or "<root>", failed_msg or "")
            return False
        self.replace(gm)
        return True

    def trace_until(self, paths, **kwargs) -> bool:
        """Trace from the top, keeping every child of ``paths`` an opaque
        leaf - the precondition of ``cut_pipeline_stage`` on those children."""
        if self.parent is not None:
            raise RuntimeError("trace_until must be called on the top schedule")
        if isinstance(paths, str):
            paths = [paths]
        leaves = list(kwargs.pop("leaf_modules", []))
        if paths == [""]:
            for name, _ in self.mod.named_children():
                leaves.append(name)
            kwargs["recursive"] = False
        else:
            for path in paths:
                for name in self[path].child:
                    leaves.append(f"{path}.{name}")
        # every level between the root and the targets is traced; siblings of
        # the targets are traced flat below their own level as usual
        return self.trace(leaf_modules=leaves, **kwargs)

    def _construct_fx_graph(self, subgraph) -> fx.GraphModule:
        """Copy a matched chain into a stand-alone GraphModule whose inputs
        are the values the chain reads from outside (in first-use order) and
        whose output is the last matched node."""
        inside = {node for _, node in subgraph}
        new_graph = fx.Graph()
        remap = {}
        for _, node in subgraph:
            for inp in node.all_input_nodes:
                if inp not in inside and inp not in remap:
                    remap[inp] = new_graph.placeholder(inp.name)
        owner = self.mod
        path = subgraph[0][0]
        if path:
            owner = self.get_module(path)
        mods = {}
        for _, node in subgraph:
            remap[node] = new_graph.node_copy(node, lambda n: remap[n])
            if node.op in ("call_module", "get_attr"):
                cur = owner
                for tok in node.target.split("."):
                    cur = getattr(cur, tok)
                mods[node.target] = cur
        new_graph.output(remap[subgraph[-1][1]])
        gm = fx.GraphModule(mods, new_graph)
        gm.graph.eliminate_dead_code()
        gm.graph.lint()
        gm.recompile()
        return gm

    def find_node(self, regex_or_pattern_fn):
        """Nodes of every traced graph below this schedule that satisfy a
        regex on ``call_module`` targets or a ``node -> bool`` predicate.
        Returns ``[(parent_module_name, node), ...]``."""
        if not isinstance(regex_or_pattern_fn, (str, Callable)):
            raise ValueError("pass a regex string or a callable node predicate")
        self.trace()
        out = []
        for name, mod in self.mod.named_modules():
            if not isinstance(mod, fx.GraphModule):
                continue
            for node in mod.graph.nodes:
                if isinstance(regex_or_pattern_fn, str):
                    if node.op == "call_module" and re.match(regex_or_pattern_fn, node.target):
                        out.append((name, node))
                elif regex_or_pattern_fn(node):
                    out.append((name, node))
        return out

    def find_subgraph(self, pattern_fn):
        """All sub-graphs matching a pattern function or ``Pattern`` module.
        Returns ``[[(parent_module_name, node), ...], ...]`` (one inner list
        per match, nodes in program order)."""
        if not isinstance(pattern_fn, (FunctionType, Pattern)):
            raise ValueError("pattern must be a function or a Pattern instance")
        self.trace()
        if isinstance(pattern_fn, Pattern):
            pattern_gm = trace_module(pattern_fn, flatten=True, leaf_modules=["ModulePattern"])
        else:
            pattern_gm = fx.symbolic_trace(pattern_fn)
        if not isinstance(pattern_gm, fx.GraphModule):
            raise RuntimeError("the pattern itself cannot be traced")
        matcher = SubgraphMatcher(pattern_gm)
        results = []
        for parent_name, submod in self.mod.named_modules():
            if not isinstance(submod, fx.GraphModule):
                continue
            target_mods = dict(submod.named_modules())
            for nodes in matcher.match_graph(submod.graph, target_mods):
                results.append([(parent_name, n) for n in nodes])
        return results

    def find(self, regex_or_pattern_fn):
        """Dispatch to ``find_node`` (regex) or ``find_subgraph`` (pattern)."""
        if isinstance(regex_or_pattern_fn, (FunctionType, Pattern)):
            return self.find_subgraph(regex_or_pattern_fn)
        if isinstance(regex_or_pattern_fn, str):
            return self.find_node(regex_or_pattern_fn)
        raise RuntimeError(f"unrecognised pattern type {type(regex_or_pattern_fn)}")


def list_primitives(name_only: bool = True):
    """Registered primitive names, or the ``{name: class}`` mapping."""
    return list(PRIMITIVES.keys()) if name_only else dict(PRIMITIVES)


def _is_leaf(module: nn.Module) -> bool:
    if getattr(module, "schedule_container", False):
        # a bare container that the hierarchical trace left between a graph and the grandchild
        # it calls ("model.decoder" called from the top graph leaves "model" such a module);
        # the containers of a flattened trace stay leaves: their members are no longer
        # schedules of their own
        return False
    mod_path = type(module).__module__
    return (mod_path.startswith("torch.nn") or mod_path.startswith("torch.ao.nn")) \
        and not isinstance(module, nn.Sequential)


def create_schedule(root: nn.Module, name: str = "", path: str = "",
                    parent: Optional[Schedule] = None, group=None, **kwargs) -> Schedule:
    """Build the schedule tree of ``root``; ``group`` is the tensor-parallel
    process group that ``shard``/``sync`` will use."""
    sch = Schedule(root, name, path, parent, group, **kwargs)
    if _is_leaf(root):
        return sch
    for child_name, child in root.named_children():
        child_path = f"{path}.{child_name}" if path else child_name
        if is_module_list(child):
            for idx, (sub_name, layer) in enumerate(child.named_children()):
                key = f"{child_name}.{sub_name}"
                sch.child[key] = create_schedule(
                    layer, key, f"{child_path}.{sub_name}", sch, group, **kwargs)
        else:
            sch.child[child_name] = create_schedule(
                child, child_name, child_path, sch, group, **kwargs)
    return sch
