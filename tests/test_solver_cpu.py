"""Sharding solver: finds the Megatron layouts for an MLP and an attention
block, prefers sequence parallelism when normalisation sits between the
blocks, and its plan runs correctly on two gloo ranks."""
import copy

import torch
import torch.nn.functional as F
from torch import nn

import slapo_b200 as slapo
from slapo_b200.parallel.solver import HardwareModel, ShardingSolver, solve_sharding

from dist_utils import run_distributed


class MLP(nn.Module):
    def __init__(self, h=64):
        super().__init__()
        self.fc1 = nn.Linear(h, 4 * h)
        self.act = nn.GELU()
        self.fc2 = nn.Linear(4 * h, h)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


class Core(nn.Module):
    """Attention core on [B, S, heads*dim] projections (whole heads shardable)."""

    def __init__(self, heads, dim):
        super().__init__()
        self.heads, self.dim = heads, dim

    def forward(self, q, k, v):
        b, s, _ = q.shape
        sp = lambda t: t.view(b, s, -1, self.dim).transpose(1, 2)  # noqa: E731
        out = F.scaled_dot_product_attention(sp(q), sp(k), sp(v))
        return out.transpose(1, 2).reshape(b, s, -1)


class Block(nn.Module):
    def __init__(self, h=64, heads=4):
        super().__init__()
        self.ln1 = nn.LayerNorm(h)
        self.q = nn.Linear(h, h)
        self.k = nn.Linear(h, h)
        self.v = nn.Linear(h, h)
        self.core = Core(heads, h // heads)
        self.o = nn.Linear(h, h)
        self.ln2 = nn.LayerNorm(h)
        self.mlp = MLP(h)

    def forward(self, x):
        y = self.ln1(x)
        x = x + self.o(self.core(self.q(y), self.k(y), self.v(y)))
        return x + self.mlp(self.ln2(x))


def _trace(model, leaf=()):
    sch = slapo.create_schedule(model, group=False)
    sch.trace(flatten=True, leaf_modules=list(leaf))
    return sch.mod


def test_mlp_gets_column_then_row_parallel():
    gm = _trace(MLP(1024))
    plan = ShardingSolver(gm, [torch.randn(8, 512, 1024)], world_size=8).solve()
    assert plan.linear == {"fc1": "S0", "fc2": "S1"}
    assert plan.finish["fc2"] in ("all_reduce", "reduce_scatter")
    assert plan.layout["fc1"] == "RS"
    assert "fc1: S0" in plan.describe()
    # replicated everywhere is what a single rank gets
    assert ShardingSolver(gm, [torch.randn(8, 512, 1024)], world_size=1).solve().linear == {}


def test_slow_link_keeps_small_layers_replicated():
    gm = _trace(MLP(64))
    slow = HardwareModel(link_bytes_per_s=1e6, collective_latency_s=1e-3)
    plan = ShardingSolver(gm, [torch.randn(2, 8, 64)], world_size=8, hardware=slow,
                          allow_token_parallel=False).solve()
    assert set(plan.linear.values()) == {"R"}


def test_block_gets_megatron_layout_and_sequence_parallel_norms():
    gm = _trace(Block(1024, 16), leaf=["Core"])
    # element-wise work made expensive (slow memory): normalisation on token shards pays
    slow_mem = HardwareModel(hbm_bytes_per_s=1e11)
    solver = ShardingSolver(gm, [torch.randn(8, 512, 1024)], world_size=8, hardware=slow_mem,
                            head_parallel_modules=(Core,), memory_weight=1e-8)
    plan = solver.solve()
    assert [plan.linear[k] for k in ("q", "k", "v", "o")] == ["S0", "S0", "S0", "S1"]
    assert plan.linear["mlp.fc1"] == "S0" and plan.linear["mlp.fc2"] == "S1"
    assert plan.layout["core"] == "RS"
    # LayerNorm between the blocks then runs on token shards when that is allowed ...
    assert plan.finish["o"] == "reduce_scatter" and plan.layout["ln2"] == "SR"
    # ... and on replicas when it is not
    plan2 = ShardingSolver(gm, [torch.randn(8, 512, 1024)], world_size=8, hardware=slow_mem,
                           head_parallel_modules=(Core,), allow_token_parallel=False,
                           memory_weight=1e-8).solve()
    assert plan2.finish["o"] == "all_reduce" and plan2.layout["ln2"] == "RR"
    assert plan.cost <= plan2.cost
    # without memory pressure the small projections are cheapest replicated on token shards
    plan3 = ShardingSolver(gm, [torch.randn(8, 512, 1024)], world_size=8,
                           head_parallel_modules=(Core,)).solve()
    assert "R" in set(plan3.linear.values())


def _apply_worker(rank, world):
    torch.manual_seed(0)
    ref = Block(64, 4)
    x = torch.randn(2, 8, 64)
    want = ref(x)
    sch = slapo.create_schedule(copy.deepcopy(ref))
    plan = solve_sharding(sch, [x], head_parallel_modules=(Core,), allow_token_parallel=False,
                          memory_weight=1.0)   # tiny model: only memory pressure makes it split
    assert plan.linear["q"] == "S0" and plan.linear["mlp.fc2"] == "S1"
    with slapo.Verify(sch, [x], device="cpu"):
        plan.apply(sch)
    model, _ = slapo.build(sch, init_weights=False)
    assert model.get_submodule("mlp.fc1").weight.shape == (256 // world, 64)
    torch.testing.assert_close(model(x), want, rtol=1e-4, atol=1e-4)


def test_plan_applies_and_verifies_on_two_ranks():
    run_distributed(_apply_worker, 2)
