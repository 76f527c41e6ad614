"""Sharding solver: choose a tensor-parallel layout for every Linear of a traced
module by dynamic programming over the dataflow graph.

Layouts of an activation ``[..., tokens, hidden]`` over ``n`` ranks (the R/S
algebra of slapo/sharding/reshard_ops.py:4-20 in the reference, which has the
layouts and their conversion costs but no solver):

* ``RR`` replicated, ``RS`` hidden axis sharded, ``SR`` token axis sharded.

Strategies of a Linear with weight ``[out, in]``:

* ``R``   weight replicated; input ``RR -> RR`` (redundant compute) or
  ``SR -> SR`` (token-parallel; weight gradients all-reduced);
* ``S0``  split ``out`` (column parallel): input ``RR`` -> output ``RS``; the
  input gradient is a partial sum, all-reduced in backward;
* ``S1``  split ``in`` (row parallel): input ``RS`` -> partial sums, finished
  by an all-reduce (``-> RR``) or a reduce-scatter over tokens (``-> SR``).

The cost of a plan is the modelled time of one forward + backward:
``FLOPs / tensor peak`` for the matmuls on each rank, ``bytes / HBM bandwidth``
for element-wise work, ``bytes over NVLink / link bandwidth`` for every
collective (layout conversions included, with their backward duals) and for
the gradient all-reduce of replicated weights that saw token shards.  The DP
runs over the nodes in topological order with the layouts of all live values
as its state - transformers keep two or three values alive, so the state
space stays tiny - and returns the cheapest assignment.  ``Plan.apply(sch)``
emits the corresponding ``shard`` / ``sync`` calls.
"""
from __future__ import annotations

import operator
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import fx, nn
from torch.fx.passes.shape_prop import ShapeProp

LAYOUTS = ("RR", "RS", "SR")

_ELEMENTWISE_FUNCS = {
    F.relu, F.gelu, F.silu, F.dropout, torch.relu, torch.tanh, torch.sigmoid, F.tanh, F.sigmoid,
    operator.neg, torch.neg,
}
_BINARY_FUNCS = {operator.add, operator.mul, operator.sub, torch.add, torch.mul, torch.sub,
                 operator.iadd, operator.truediv}
_ELEMENTWISE_MODS = (nn.ReLU, nn.GELU, nn.SiLU, nn.Dropout, nn.Tanh, nn.Sigmoid, nn.Identity)
_LAST_DIM_MODS = (nn.LayerNorm, nn.Softmax)
_VIEW_METHODS = {"view", "reshape", "permute", "transpose", "contiguous", "to", "type", "float",
                 "bfloat16", "half"}


@dataclass
class HardwareModel:
    """Rates used to turn FLOPs and bytes into seconds (defaults: one B200 and
    its NVLink 5 port as measured with cuBLAS, a device copy and a peer copy)."""
    flops: float = 1.4e15
    hbm_bytes_per_s: float = 6.4e12
    link_bytes_per_s: float = 7.7e11
    collective_latency_s: float = 8e-6


@dataclass
class Plan:
    world_size: int
    cost: float
    linear: dict = field(default_factory=dict)      # module path -> "R" | "S0" | "S1"
    finish: dict = field(default_factory=dict)      # S1 module path -> "all_reduce" | "reduce_scatter"
    layout: dict = field(default_factory=dict)      # node name -> layout of its output
    reshards: list = field(default_factory=list)    # (consumer node name, producer node name, "XX->YY")
    token_axis: int = 1

    def describe(self):
        rows = [f"plan for {self.world_size} ranks, modelled step time {self.cost * 1e6:.1f} us"]
        for path, strat in self.linear.items():
            extra = f" + {self.finish[path]}" if path in self.finish else ""
            rows.append(f"  {path}: {strat}{extra}")
        for consumer, producer, scheme in self.reshards:
            rows.append(f"  reshard {scheme} between {producer} and {consumer}")
        return "\n".join(rows)

    def apply(self, sch, graph_module=None):
        """Emit ``shard`` / ``sync`` on ``sch`` (whose module paths are the
        ``call_module`` targets the plan was solved for)."""
        for path, strat in self.linear.items():
            sub = sch[path]
            has_bias = getattr(sub.mod, "bias", None) is not None
            if strat == "S0":
                sub.shard("weight", axis=0)
                if has_bias:
                    sub.shard("bias", axis=0)
                sub.sync("bwd_post", "all_reduce")
            elif strat == "S1":
                sub.shard("weight", axis=1)
                if self.finish[path] == "all_reduce":
                    sub.sync("fwd_post", "all_reduce")
                else:
                    sub.sync("fwd_post", "reduce_scatter", axis=self.token_axis)
            elif strat == "R" and self.layout.get(path) == "SR":
                for name in ("weight", "bias"):
                    if getattr(sub.mod, name, None) is not None:
                        sub.annotate(name, "replicated_param", True)
        for consumer, producer, scheme in self.reshards:
            if consumer in sch:
                sch[consumer].sync("fwd_pre", scheme)
            elif producer in sch:
                sch[producer].sync("fwd_post", scheme)
            else:
                raise RuntimeError(f"reshard {scheme} between {producer} and {consumer} has no "
                                   "module to attach a hook to; trace with those ops as modules")
        return sch


class ShardingSolver:
    def __init__(self, gm: fx.GraphModule, example_inputs, world_size: int, hardware=None,
                 bytes_per_elem: int = 2, token_axis: int = 1, output_layout: str = "RR",
                 head_parallel_modules=(), allow_token_parallel=True, memory_weight=0.0):
        self.gm = gm
        self.n = world_size
        self.hw = hardware or HardwareModel()
        self.bpe = bytes_per_elem
        self.token_axis = token_axis
        self.output_layout = output_layout
        self.head_parallel = tuple(head_parallel_modules)
        self.layouts = LAYOUTS if allow_token_parallel else ("RR", "RS")
        # seconds charged per byte of parameter resident on a rank: 0 optimises time only
        # (small models then stay replicated and run token-parallel); a positive value
        # expresses memory pressure and pushes large weights to be split
        self.memory_weight = memory_weight
        ShapeProp(gm).propagate(*example_inputs)
        self.mods = dict(gm.named_modules())

    # ---- sizes and costs ------------------------------------------------ #
    @staticmethod
    def _numel(node):
        meta = node.meta.get("tensor_meta")
        if meta is None or not hasattr(meta, "shape"):
            return 0
        n = 1
        for s in meta.shape:
            n *= s
        return n

    def _bytes(self, node):
        return self._numel(node) * self.bpe

    def _link(self, nbytes, factor):
        """Time of a collective moving ``factor * (n-1)/n * nbytes`` per rank."""
        if nbytes == 0 or factor == 0:
            return 0.0
        moved = factor * nbytes * (self.n - 1) / self.n
        return self.hw.collective_latency_s + moved / self.hw.link_bytes_per_s

    def reshard_cost(self, src, dst, nbytes):
        """Forward + backward time of converting a value's layout."""
        if src == dst:
            return 0.0
        pair = {src, dst}
        if "RR" in pair:
            # one direction is a slice (free) and the other an all-gather, in forward
            # for "-> RR" and in backward for "RR ->": one gather-sized transfer
            return self._link(nbytes, 1.0)
        # RS <-> SR: all-to-all forward and backward, each moving 1/n of the shard
        return 2 * self._link(nbytes / self.n, 1.0)

    def _elementwise(self, nbytes, layout, n_tensors=2):
        share = 1.0 if layout == "RR" else 1.0 / self.n
        return 3 * n_tensors * nbytes * share / self.hw.hbm_bytes_per_s  # fwd + ~2x bwd traffic

    # ---- per-node options ------------------------------------------------ #
    def _linear_options(self, node, mod):
        """[(strategy, finish, required input layout, output layout, cost)]"""
        x = node.all_input_nodes[0]
        tokens = self._numel(x) // max(mod.in_features, 1)
        flops = 3 * 2 * tokens * mod.in_features * mod.out_features  # fwd + dgrad + wgrad
        w_bytes = mod.weight.numel() * self.bpe
        in_bytes, out_bytes = self._bytes(x), self._bytes(node)
        t_full = flops / self.hw.flops
        m_full = w_bytes * self.memory_weight
        m_part = m_full / self.n
        opts = [("R", None, "RR", "RR", t_full + m_full)]
        if "SR" in self.layouts:
            opts.append(("R", None, "SR", "SR", t_full / self.n + self._link(w_bytes, 2.0) + m_full))
        if mod.out_features % self.n == 0:
            opts.append(("S0", None, "RR", "RS",
                         t_full / self.n + self._link(in_bytes, 2.0) + m_part))
        if mod.in_features % self.n == 0:
            opts.append(("S1", "all_reduce", "RS", "RR",
                         t_full / self.n + self._link(out_bytes, 2.0) + m_part))
            if "SR" in self.layouts:
                opts.append(("S1", "reduce_scatter", "RS", "SR",
                             t_full / self.n + 2 * self._link(out_bytes, 1.0) + m_part))
        return opts

    def _options(self, node):
        """Generic form: list of (tag, [required layout per input], output layout, cost)."""
        ins = node.all_input_nodes
        nbytes = self._bytes(node)
        if node.op == "placeholder" or node.op == "get_attr":
            return [(None, [], "RR", 0.0)]
        if node.op == "output":
            return [(None, [self.output_layout] * len(ins), self.output_layout, 0.0)]
        if node.op == "call_module":
            mod = self.mods[node.target]
            if isinstance(mod, nn.Linear):
                return [((s, f), [need], out, c) for s, f, need, out, c in self._linear_options(node, mod)]
            if isinstance(mod, _LAST_DIM_MODS):
                allowed = [l for l in self.layouts if l != "RS"]
                return [(None, [l] * len(ins), l, self._elementwise(nbytes, l)) for l in allowed]
            if isinstance(mod, _ELEMENTWISE_MODS):
                return [(None, [l] * len(ins), l, self._elementwise(nbytes, l)) for l in self.layouts]
            if isinstance(mod, self.head_parallel) and self.head_parallel:
                # attention core on [.., heads*dim] projections: whole heads per rank, or replicated
                return [(None, [l] * len(ins), l, self._elementwise(nbytes, l, 4)) for l in ("RR", "RS")]
            return [(None, ["RR"] * len(ins), "RR", self._elementwise(nbytes, "RR"))]
        if node.op == "call_function":
            if node.target in _BINARY_FUNCS or node.target in _ELEMENTWISE_FUNCS:
                return [(None, [l] * len(ins), l, self._elementwise(nbytes, l)) for l in self.layouts]
            if node.target in (F.layer_norm, F.softmax, torch.softmax):
                allowed = [l for l in self.layouts if l != "RS"]
                return [(None, [l] * len(ins), l, self._elementwise(nbytes, l)) for l in allowed]
            if node.target is operator.getitem:
                return [(None, [l] * len(ins), l, 0.0) for l in self.layouts]
        if node.op == "call_method" and node.target in _VIEW_METHODS:
            return [(None, [l] * len(ins), l, 0.0) for l in ("RR", "RS")]
        return [(None, ["RR"] * len(ins), "RR", self._elementwise(nbytes, "RR"))]

    # ---- the DP ---------------------------------------------------------- #
    def solve(self) -> Plan:
        if self.n == 1:
            return Plan(1, 0.0, token_axis=self.token_axis)
        nodes = list(self.gm.graph.nodes)
        last_use = {}
        for idx, node in enumerate(nodes):
            for inp in node.all_input_nodes:
                last_use[inp] = idx
        # state: tuple of (node index, layout) of live values -> (cost, trace)
        states = {(): (0.0, ())}
        index = {node: i for i, node in enumerate(nodes)}
        for idx, node in enumerate(nodes):
            options = self._options(node)
            new_states = {}
            for state, (cost, trace) in states.items():
                live = dict(state)
                for tag, needs, out_layout, op_cost in options:
                    total = cost + op_cost
                    moves = []
                    for inp, need in zip(node.all_input_nodes, needs):
                        have = live[index[inp]]
                        if not self._numel(inp):      # non-tensor value: nothing to convert
                            continue
                        if have != need:
                            total += self.reshard_cost(have, need, self._bytes(inp))
                            moves.append((node.name, inp.name, f"{have}->{need}"))
                    nxt = {k: v for k, v in live.items() if last_use.get(nodes[k], -1) > idx}
                    if last_use.get(node, -1) > idx:
                        nxt[idx] = out_layout
                    key = tuple(sorted(nxt.items()))
                    entry = (total, trace + ((node, tag, out_layout, tuple(moves)),))
                    if key not in new_states or total < new_states[key][0]:
                        new_states[key] = entry
            states = new_states
        cost, trace = min(states.values(), key=lambda e: e[0])
        plan = Plan(self.n, cost, token_axis=self.token_axis)
        for node, tag, layout, moves in trace:
            plan.layout[str(node.target) if node.op == "call_module" else node.name] = layout
            if tag is not None:
                strat, finish = tag
                plan.linear[node.target] = strat
                if finish is not None:
                    plan.finish[node.target] = finish
            for consumer, producer, scheme in moves:
                cons = next(n for n in nodes if n.name == consumer)
                prod = next(n for n in nodes if n.name == producer)
                plan.reshards.append((cons.target if cons.op == "call_module" else cons.name,
                                      prod.target if prod.op == "call_module" else prod.name,
                                      scheme))
        return plan


def solve_sharding(sch, example_inputs, hardware=None, **kwargs) -> Plan:
    """Solve for ``sch.world_size`` ranks on a flattened trace of a *copy* of
    the module (so that every Linear is visible in one graph while ``sch``
    keeps its hierarchy for :meth:`Plan.apply`) and return the :class:`Plan`."""
    import copy

    from ..schedule import create_schedule

    probe = create_schedule(copy.deepcopy(sch.mod), group=False)
    probe.trace(flatten=True,
                leaf_modules=[c.__name__ for c in kwargs.get("head_parallel_modules", ())])
    gm = probe.mod
    if not isinstance(gm, fx.GraphModule):
        raise RuntimeError("the module could not be traced; the solver needs a dataflow graph")
    solver = ShardingSolver(gm, example_inputs, sch.world_size, hardware, **kwargs)
    return solver.solve()
