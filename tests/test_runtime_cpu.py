"""Checkpoint with RNG replay, fork_rng, seeding rules, meta-device init +
consolidation, Verify (must fail on a missing sync) - CPU / gloo."""
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn

import slapo_b200 as slapo
from slapo_b200.random import get_cuda_rng_tracker, is_random_seed_set, set_random_seed

from dist_utils import run_distributed


class DropBlock(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(32, 32)
        self.drop_tp = nn.Dropout(0.5)     # runs inside the tensor-parallel RNG stream
        self.fc2 = nn.Linear(32, 32)
        self.drop = nn.Dropout(0.5)        # default stream

    def forward(self, x):
        with get_cuda_rng_tracker().fork():
            h = self.drop_tp(self.fc1(x))
        return self.drop(self.fc2(h))


def test_checkpoint_replays_both_rng_streams():
    set_random_seed(123, tp_rank=0)
    torch.manual_seed(0)
    model = DropBlock()
    x = torch.randn(4, 32, requires_grad=True)

    def run(mod):
        set_random_seed(123, tp_rank=0)
        x.grad = None
        for p in mod.parameters():
            p.grad = None
        out = mod(x)
        out.sum().backward()
        inner = mod.mod if hasattr(mod, "mod") else mod      # un-wrap the checkpoint wrapper
        return out.detach().clone(), x.grad.clone(), inner.fc1.weight.grad.clone()

    ref = run(model)
    sch = slapo.create_schedule(copy.deepcopy(model))
    sch.checkpoint()
    ckpt_model, _ = slapo.build(sch, init_weights=False)
    got = run(ckpt_model)
    for a, b in zip(ref, got):
        assert torch.equal(a, b)        # bit-exact: the recompute saw the same masks


def test_checkpoint_function_api():
    lin = nn.Linear(8, 8)
    x = torch.randn(2, 8, requires_grad=True)
    out = slapo.checkpoint(lambda t: torch.relu(lin(t)), x)
    out.sum().backward()
    g = x.grad.clone()
    x.grad = None
    torch.relu(lin(x)).sum().backward()
    torch.testing.assert_close(g, x.grad)


def test_seed_rules():
    base = set_random_seed(2013, dp_rank=1, pp_rank=2, tp_rank=3)
    assert base == 2013 + 200 + 10
    assert is_random_seed_set()
    states = get_cuda_rng_tracker().get_states()
    assert len(states) == 1
    # default stream follows the base seed unless always_enable_tp_seed
    set_random_seed(7, tp_rank=1)
    a = torch.rand(3)
    torch.manual_seed(7)
    torch.testing.assert_close(a, torch.rand(3))
    set_random_seed(7, tp_rank=1, always_enable_tp_seed=True)
    a = torch.rand(3)
    torch.manual_seed(7 + 2718 + 1)
    torch.testing.assert_close(a, torch.rand(3))
    # the tensor-parallel stream is seeded with seed + 2718 + tp_rank
    set_random_seed(7, tp_rank=1)
    with get_cuda_rng_tracker().fork():
        b = torch.rand(3)
    torch.manual_seed(7 + 2718 + 1)
    torch.testing.assert_close(b, torch.rand(3))


def _fork_rng_worker(rank, world):
    set_random_seed(99, tp_rank=rank)
    drop = nn.Dropout(0.5)
    x = torch.ones(64, 64)
    same = drop(x)
    gathered = [torch.empty_like(same) for _ in range(world)]
    dist.all_gather(gathered, same)
    assert torch.equal(gathered[0], gathered[1])         # without fork_rng: identical masks
    sch = slapo.create_schedule(nn.Sequential(nn.Dropout(0.5)))
    sch["0"].fork_rng()
    out = sch.mod(x)
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    assert not torch.equal(gathered[0], gathered[1])     # with fork_rng: per-rank masks


def test_fork_rng_differs_across_tp_ranks():
    run_distributed(_fork_rng_worker, 2)


# ---------------------------------------------------------------------- #
class Wide(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(16, 64)
        self.fc2 = nn.Linear(64, 16)

    def forward(self, x):
        return self.fc2(torch.relu(self.fc1(x)))


def _consolidation_worker(rank, world):
    with slapo.init_empty_weights():
        model = Wide()
    assert model.fc1.weight.is_meta
    sch = slapo.create_schedule(model)
    sch["fc1"].shard("weight", axis=0)
    sch["fc1"].shard("bias", axis=0)
    sch["fc1"].sync("bwd_post", "all_reduce")
    sch["fc2"].shard("weight", axis=1)
    sch["fc2"].sync("fwd_post", "all_reduce")
    assert sch.mod.fc1.weight.is_meta and sch.mod.fc1.weight.shape == (32, 16)

    def init(mod):
        if isinstance(mod, nn.Linear):
            # rank-dependent on purpose: consolidation must spread rank 0's values
            nn.init.constant_(mod.weight, 1.0 + rank)
            nn.init.zeros_(mod.bias)
            with torch.no_grad():
                mod.weight[0, 0] = 5.0      # full-tensor coordinates: only rank 0's shard sees it

    built, _ = slapo.build(sch, init_weights=init)
    assert not built.fc1.weight.is_meta and built.fc1.weight.shape == (32, 16)
    # every rank holds a slice of rank 0's full tensor
    assert float(built.fc1.weight[1, 1]) == 1.0
    assert float(built.fc1.weight[0, 0]) == (5.0 if rank == 0 else 1.0)
    assert float(built.fc2.weight[0, 0]) == (5.0 if rank == 0 else 1.0)
    out = built(torch.ones(2, 16))
    ref = torch.relu(torch.ones(2, 16) @ torch.ones(16, 64))  # apart from the marked element
    assert out.shape == (2, 16) and torch.isfinite(out).all() and ref.shape == (2, 64)


def test_meta_init_and_consolidation():
    run_distributed(_consolidation_worker, 2)


def test_build_init_weights_false_keeps_materialised_params():
    model = Wide()
    w = model.fc1.weight.detach().clone()
    sch = slapo.create_schedule(model)
    built, opt = slapo.build(sch, init_weights=False)
    assert opt is None
    torch.testing.assert_close(built.fc1.weight, w)


# ---------------------------------------------------------------------- #
def _verify_worker(rank, world):
    model = Wide()
    sch = slapo.create_schedule(model)
    with slapo.Verify(sch, [torch.randn(4, 16)], device="cpu"):
        sch["fc1"].shard("weight", axis=0)
        sch["fc1"].shard("bias", axis=0)
        sch["fc1"].sync("bwd_post", "all_reduce")
        sch["fc2"].shard("weight", axis=1)
        sch["fc2"].sync("fwd_post", "all_reduce")

    sch = slapo.create_schedule(Wide())
    with pytest.raises(Exception):
        with slapo.Verify(sch, [torch.randn(4, 16)], device="cpu"):
            sch["fc1"].shard("weight", axis=0)
            sch["fc1"].shard("bias", axis=0)
            sch["fc2"].shard("weight", axis=1)     # the all_reduce after fc2 is missing

    # gradients are checked too: forward is right, the input gradient is not reduced
    sch = slapo.create_schedule(Wide())
    x = torch.randn(4, 16, requires_grad=True)
    with pytest.raises(Exception):
        with slapo.Verify(sch, [x], device="cpu"):
            sch["fc1"].shard("weight", axis=0)
            sch["fc1"].shard("bias", axis=0)
            sch["fc2"].shard("weight", axis=1)
            sch["fc2"].sync("fwd_post", "all_reduce")   # bwd_post all_reduce on fc1 missing


def test_verify_passes_and_fails():
    run_distributed(_verify_worker, 2)


def test_verify_disabled_is_a_no_op():
    sch = slapo.create_schedule(Wide())
    with slapo.Verify(sch, [torch.randn(2, 16)], enable=False):
        sch["fc1"].replace(nn.Linear(16, 64))
