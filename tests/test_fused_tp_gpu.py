"""Fused GEMM+collective kernels, exercised on ONE GPU: the ranks of a group
are impersonated one after the other with the peers' flags pre-set (never two
mutually waiting kernels on a device).  Reference = fp32 matmuls on the
gathered operands."""
import pytest
import torch

from slapo_b200.ops import native
from slapo_b200.parallel import fused_tp as ft
from slapo_b200.parallel.symm import LocalSymmContext

pytestmark = pytest.mark.gpu


def _put(ctx, rank, name, t):
    """Fill fake rank ``rank``'s symmetric buffer ``name`` with ``t``."""
    buf = ctx.as_rank(rank).buffer(name, t.numel() * t.element_size())
    buf.view(t.dtype, tuple(t.shape)).copy_(t)


def _close(a, b, k, tol=2e-2):
    scale = max(1.0, k ** 0.5)
    torch.testing.assert_close(a.float() / scale, b.float() / scale, rtol=tol, atol=tol)


@pytest.mark.parametrize("world,n", [(2, 320), (4, 320), (8, 384), (8, 512)])
def test_all_gather_gemm(world, n):
    torch.manual_seed(0)
    ts, k = 256, 192
    ctx = LocalSymmContext(world)
    shards = [torch.randn(ts, k, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    w = [torch.randn(n, k, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    bias = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    for r in range(world):
        _put(ctx, r, "ag_in", shards[r])
    full = torch.cat(shards, 0).float()
    for r in range(world):
        ctx.as_rank(r)
        ctx.preset_flags(ctx.epoch + 1)
        y = ft.ag_gemm(ctx, shards[r], w[r], bias, staged=ctx.buffer("ag_in", ts * k * 2))
        assert native.ops().device_status() == 0
        _close(y, full @ w[r].float().t() + bias.float(), k)


@pytest.mark.parametrize("world,n,ts", [(2, 320, 256), (4, 192, 384), (8, 384, 128)])
@pytest.mark.parametrize("keep", [False, True])
@pytest.mark.parametrize("mode", ["push", "gather"])
def test_all_gather_gemm_pushed(world, n, ts, keep, mode):
    """Pushed gather: the emulated rank stores its own rows into every rank's staging slot
    (rank by rank here, the emulation has no multicast address) and multiplies the gathered
    operand; the other owners' rows and block flags are put into its slot beforehand.
    ``push``: inside the GEMM kernel; ``gather``: push kernel, then the pair GEMM."""
    torch.manual_seed(1)
    k = 192
    t = ts * world
    ctx = LocalSymmContext(world)
    shards = [torch.randn(ts, k, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    w = [torch.randn(n, k, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    bias = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    full = torch.cat(shards, 0)
    nbytes = t * k * 2
    name = f"ag_slot_{nbytes}_0"
    for r in range(world):
        ctx.as_rank(r).buffer(name, ft.RECV_HEADER_BYTES + nbytes)
    hdr = ft.RECV_HEADER_BYTES

    def data(q):
        return ctx._buffers[name][q][hdr:hdr + nbytes].view(torch.bfloat16).view(t, k)

    for r in range(world):
        ctx.as_rank(r)
        for q in range(world):
            data(q).copy_(full)
            data(q)[r * ts:(r + 1) * ts].zero_()          # what rank r has to deliver
        # 16 flag words per 128-row block (one per 8-row slice)
        flags = ctx._buffers[name][r][:t // 128 * 64].view(torch.int32)
        flags.fill_(ctx.epoch + 1)                         # the other owners' blocks "arrived"
        flags[r * (ts // 128) * 16:(r + 1) * (ts // 128) * 16] = 0
        ctx.preset_flags(ctx.epoch + 1, ready=True, done=True)   # "gather" also waits for done
        y, gathered, token = ft.ag_gemm_pushed(ctx, shards[r], w[r], bias, keep=keep, mode=mode)
        assert native.ops().device_status() == 0
        _close(y, full.float() @ w[r].float().t() + bias.float(), k)
        for q in range(world):
            assert torch.equal(data(q), full), f"rank {r}'s rows in rank {q}'s slot"
            if mode == "push":      # the fused kernel raises a flag per 8-row slice
                fl = ctx._buffers[name][q][:t // 128 * 64].view(torch.int32)
                assert bool((fl[r * (ts // 128) * 16:(r + 1) * (ts // 128) * 16] == ctx.epoch).all())
        if keep:
            assert token == (nbytes, 0) and torch.equal(gathered, full)
            ft.stage_pool(ctx).release(token)
        else:
            assert gathered is None and token is None


def test_stage_pool_is_deterministic_and_bounded(monkeypatch):
    """Slots come from a LIFO free list per size; beyond the byte limit `acquire` refuses and
    the caller falls back to the transient slot; `release_all` returns what was never released."""
    monkeypatch.setenv("SLAPO_B200_AG_POOL_GB", str(3 * 2**20 / 2**30))
    ctx = LocalSymmContext(2)
    pool = ft.StagePool(ctx)
    a, b, c = (pool.acquire(2**20) for _ in range(3))
    assert [x[0] for x in (a, b, c)] == [(2**20, 0), (2**20, 1), (2**20, 2)]
    assert pool.acquire(2**20) is None
    pool.release(b[0])
    pool.release(b[0])                                      # a second release is ignored
    assert pool.acquire(2**20)[0] == (2**20, 1)
    pool.release_all()
    assert sorted(pool.free[2**20]) == [0, 1, 2]
    assert pool.acquire(2**20)[0] == (2**20, 0)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode", ["rs", "ar"])
def test_gemm_reduce_scatter_and_all_reduce(world, mode):
    torch.manual_seed(1)
    t, kl, n = 128 * world * 2, 128, 256
    ctx = LocalSymmContext(world)
    x = [torch.randn(t, kl, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    w = [torch.randn(n, kl, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    bias = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    partials = [x[r].float() @ w[r].float().t() for r in range(world)]
    # the reduction sums 16-bit partials, like the kernel
    total = sum(p.to(torch.bfloat16).float() for p in partials) + bias.float()
    outs = [None] * world
    recv_name = "rs_recv" if mode == "rs" else "ar_recv"
    ctx.buffer(recv_name, ft.RECV_HEADER_BYTES + t * n * 2)   # exists before the flags are preset
    for sweep in range(2):  # sweep 0 fills every receive slot, sweep 1 reduces real data
        for r in range(world):
            ctx.as_rank(r)
            ctx.preset_flags(ctx.epoch + 1, ready=True, done=True, done2=True)
            ctx.preset_block_flags(recv_name, ctx.epoch + 1, t // world // 128)
            if mode == "rs":
                outs[r] = ft.gemm_rs(ctx, x[r], w[r], bias)
            else:
                outs[r] = ft.gemm_ar(ctx, x[r], w[r], bias)
            assert native.ops().device_status() == 0
    rows = t // world
    for r in range(world):
        if mode == "rs":
            _close(outs[r], total[r * rows:(r + 1) * rows], kl * world)
        else:
            # a fake rank only receives its own reduced rows in its output buffer
            _close(outs[r][r * rows:(r + 1) * rows], total[r * rows:(r + 1) * rows], kl * world)


def test_gathered_contraction_weight_gradients():
    """dW = dY^T all_gather(X) (B gathered along K) and dW = all_gather(dY)^T X
    (A gathered along K)."""
    torch.manual_seed(2)
    world, ts, k, n = 2, 128, 192, 128
    t = ts * world
    ctx = LocalSymmContext(world)
    xs = [torch.randn(ts, k, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    dy = torch.randn(t, n, device="cuda", dtype=torch.bfloat16)
    for r in range(world):
        _put(ctx, r, "xs", xs[r])
    ctx.as_rank(0)
    ctx.preset_flags(ctx.epoch + 1)
    staged = ctx.buffer("xs", ts * k * 2)
    dw = torch.empty(n, k, device="cuda", dtype=torch.bfloat16)
    ft.comm_gemm(ctx, a_ptrs=[dy.data_ptr()], b_ptrs=staged.ptrs(), M=n, N=k, K=t, lda=n, ldb=k,
                 a_mn=True, b_mn=True, dtype=dy.dtype, gather=ft.GATHER_B_K, seg_len=ts,
                 out_ptr=dw.data_ptr(), ldo=k)
    assert native.ops().device_status() == 0
    _close(dw, dy.float().t() @ torch.cat(xs, 0).float(), t)
    # A gathered along the contraction
    dys = [torch.randn(ts, n, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    x = torch.randn(t, k, device="cuda", dtype=torch.bfloat16)
    for r in range(world):
        _put(ctx, r, "dys", dys[r])
    ctx.as_rank(1)
    ctx.preset_flags(ctx.epoch + 1)
    staged = ctx.buffer("dys", ts * n * 2)
    dw2 = torch.empty(n, k, device="cuda", dtype=torch.bfloat16)
    ft.comm_gemm(ctx, a_ptrs=staged.ptrs(), b_ptrs=[x.data_ptr()], M=n, N=k, K=t, lda=n, ldb=k,
                 a_mn=True, b_mn=True, dtype=x.dtype, gather=ft.GATHER_A_K, seg_len=ts,
                 out_ptr=dw2.data_ptr(), ldo=k)
    assert native.ops().device_status() == 0
    _close(dw2, torch.cat(dys, 0).float().t() @ x.float(), t)


def test_missing_peer_times_out_cleanly():
    """A peer that never shows up: the bounded wait runs out, the kernel sets
    the status word and returns; the context stays usable."""
    world, ts, k, n = 2, 128, 64, 64
    ctx = LocalSymmContext(world, wait_seconds=0.02)
    xs = torch.randn(ts, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    _put(ctx, 0, "ag_in", xs)
    _put(ctx, 1, "ag_in", xs)
    ctx.as_rank(0)  # flags of rank 1 are NOT set
    ft.ag_gemm(ctx, xs, w, None, staged=ctx.buffer("ag_in", ts * k * 2))
    torch.cuda.synchronize()
    assert native.ops().device_status() == 4
    # the device is fine afterwards
    ctx.preset_flags(ctx.epoch + 1)
    y = ft.ag_gemm(ctx, xs, w, None, staged=ctx.buffer("ag_in", ts * k * 2))
    assert native.ops().device_status() == 0
    _close(y, torch.cat([xs, xs], 0).float() @ w.float().t(), k)
    # the pushed forms wait for every rank to enter before they write anybody's slot
    for mode in ("push", "gather"):
        ft.ag_gemm_pushed(ctx, xs, w, mode=mode)
        torch.cuda.synchronize()
        assert native.ops().device_status() == 4
