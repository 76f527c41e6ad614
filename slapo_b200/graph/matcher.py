"""Dataflow sub-graph matcher used by ``Schedule.find``.

The pattern is an fx graph (traced from a pattern function or a ``Pattern``
module).  A match maps every compute node of the pattern to a distinct node
of the target graph such that

* the two nodes are *compatible*: same op and target; a functional call in
  the pattern against a module call of the equivalent class (``F.relu`` vs
  ``nn.ReLU``); ``call_module(regex, ...)`` or a ``ModulePattern`` child
  against any module call whose name matches the regex; a typed child of a
  ``Pattern`` against a module call of exactly that class; and
* every data edge of the pattern exists in the target: if pattern node ``b``
  consumes pattern node ``a`` then the image of ``b`` consumes the image of
  ``a``.

The search anchors the first pattern node on each target node in program
order and extends the mapping by depth-first search with backtracking; a
target node joins at most one match.  The reference implementation
(slapo/schedule.py:255-398) scans the node list greedily and compares only
operator kinds; requiring the data edges removes its false positives while
accepting every case its tests describe (chains, trees, diamonds, two-path
and horizontal patterns).
"""
from __future__ import annotations

import re

from torch import fx

from ..pattern import ModulePattern, call_module
from ..utils.mapping import MAPPING_FROM_FUNCTIONAL_TO_MODULE


def _pattern_nodes(pattern_gm: fx.GraphModule):
    return [n for n in pattern_gm.graph.nodes if n.op not in ("placeholder", "output")]


class SubgraphMatcher:
    def __init__(self, pattern_gm: fx.GraphModule):
        self.pattern_gm = pattern_gm
        self.pattern_mods = dict(pattern_gm.named_modules())
        self.pnodes = _pattern_nodes(pattern_gm)
        if not self.pnodes:
            raise RuntimeError("the pattern has no compute node")

    # ------------------------------------------------------------------ #
    def compatible(self, pnode: fx.Node, gnode: fx.Node, target_mods) -> bool:
        if gnode.op in ("placeholder", "output"):
            return False
        if pnode.op == "call_function" and pnode.target is call_module:
            return gnode.op == "call_module" and re.match(pnode.args[0], gnode.target) is not None
        if pnode.op == gnode.op and pnode.op in ("call_function", "call_method"):
            return pnode.target == gnode.target
        if pnode.op == "call_function" and gnode.op == "call_module":
            cls = MAPPING_FROM_FUNCTIONAL_TO_MODULE.get(pnode.target)
            return cls is not None and type(target_mods.get(gnode.target)) is cls
        if pnode.op == "call_module" and gnode.op == "call_module":
            pmod = self.pattern_mods.get(pnode.target)
            if isinstance(pmod, ModulePattern):
                return re.match(pmod.name, gnode.target) is not None
            return type(pmod) is type(target_mods.get(gnode.target))
        if pnode.op == "call_module" and gnode.op == "call_function":
            pmod = self.pattern_mods.get(pnode.target)
            return MAPPING_FROM_FUNCTIONAL_TO_MODULE.get(gnode.target) is type(pmod)
        if pnode.op == "get_attr" and gnode.op == "get_attr":
            return True
        return False

    @staticmethod
    def _pattern_inputs(pnode):
        return [a for a in pnode.all_input_nodes if a.op != "placeholder"]

    def _extend(self, idx, mapping, used, gnodes_after, target_mods):
        if idx == len(self.pnodes):
            return True
        pnode = self.pnodes[idx]
        deps = self._pattern_inputs(pnode)
        if deps:
            # candidates: consumers of an already-mapped producer
            cands = list(mapping[deps[0]].users)
        else:
            cands = gnodes_after
        for g in cands:
            if g in used or g in mapping.values():
                continue
            if not self.compatible(pnode, g, target_mods):
                continue
            g_inputs = set(g.all_input_nodes)
            if any(mapping[d] not in g_inputs for d in deps):
                continue
            mapping[pnode] = g
            if self._extend(idx + 1, mapping, used, gnodes_after, target_mods):
                return True
            del mapping[pnode]
        return False

    def match_graph(self, graph: fx.Graph, target_mods, used=None):
        """All non-overlapping matches inside one graph, in program order."""
        used = set() if used is None else used
        nodes = list(graph.nodes)
        order = {n: i for i, n in enumerate(nodes)}
        results = []
        first = self.pnodes[0]
        for i, g in enumerate(nodes):
            if g in used or not self.compatible(first, g, target_mods):
                continue
            mapping = {first: g}
            if self._extend(1, mapping, used, nodes[i + 1:], target_mods):
                matched = [mapping[p] for p in self.pnodes]
                matched.sort(key=lambda n: order[n])
                used.update(matched)
                results.append(matched)
        return results
