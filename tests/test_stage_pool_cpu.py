"""Host-side logic of the pushed all-gather: the staging-slot pool hands out slots by a
deterministic rule (every rank of a group must pick the same slot for the same operation), and
the mode selection follows the context and the environment."""
import pytest

from slapo_b200.parallel import fused_tp as ft


class _Ctx:
    """Stands in for a symmetric-memory context: remembers which buffers were asked for."""

    def __init__(self, world=4, nvls=True):
        self.world, self.rank, self.nvls = world, 0, nvls
        self.asked = []

    def buffer(self, name, nbytes):
        self.asked.append((name, nbytes))
        return (name, nbytes)


def test_two_ranks_pick_the_same_slots(monkeypatch):
    monkeypatch.setenv("SLAPO_B200_AG_POOL_GB", "1")
    seqs = []
    for _ in range(2):                        # two "ranks" running the same program
        pool = ft.StagePool(_Ctx())
        seq = []
        held = []
        for step in range(3):
            for layer in range(4):            # forward: keep one slot per layer
                token, buf = pool.acquire(1 << 20)
                held.append(token)
                seq.append(buf[0])
                t2, b2 = pool.acquire(1 << 20)   # a transient use in between
                seq.append(b2[0])
                pool.release(t2)
            while held:                       # backward: release in reverse order
                pool.release(held.pop())
        seqs.append(seq)
    assert seqs[0] == seqs[1]
    assert len(set(seqs[0])) == 5             # four kept slots + one transient, reused every step


def test_pool_limit_and_release_all(monkeypatch):
    monkeypatch.setenv("SLAPO_B200_AG_POOL_GB", str(2.5 * 2**20 / 2**30))
    ctx = _Ctx()
    pool = ft.StagePool(ctx)
    a = pool.acquire(1 << 20)
    b = pool.acquire(1 << 20)
    assert a[0] == (1 << 20, 0) and b[0] == (1 << 20, 1)
    assert pool.acquire(1 << 20) is None                        # 3 MiB would exceed the limit
    assert pool.transient(1 << 20)[0] == f"ag_slot_{1 << 20}_t"
    assert ctx.asked[-1][1] == ft.RECV_HEADER_BYTES + (1 << 20)   # header + operand
    pool.release(None)                                           # the transient slot has no token
    ft.step_boundary()                                           # returns what was never released
    assert not pool.out and pool.acquire(1 << 20)[0] == (1 << 20, 0)


@pytest.mark.parametrize("env,nvls,want", [(None, True, "gather"), (None, False, "pull"),
                                           ("push", False, "push"), ("pull", True, "pull"),
                                           ("bogus", True, "gather")])
def test_all_gather_mode_selection(monkeypatch, env, nvls, want):
    if env is None:
        monkeypatch.delenv("SLAPO_B200_AG_MODE", raising=False)
    else:
        monkeypatch.setenv("SLAPO_B200_AG_MODE", env)
    ctx = _Ctx(nvls=nvls)
    assert ft.ag_mode(ctx) == want
    assert ft.push_enabled(ctx) == (want != "pull")
    # whole 128-row blocks, at most 1024 of them in the gathered operand
    assert ft._can_push(ctx, 16384) == (want != "pull")
    assert not ft._can_push(ctx, 100) and not ft._can_push(_Ctx(world=8, nvls=True), 16384 + 128)
