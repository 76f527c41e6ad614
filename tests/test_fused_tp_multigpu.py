"""Fused TP linears on real peers: 2+ GPUs, NCCL bootstrap, symmetric memory.
Compared with the gathered fp32 reference, forward and backward."""

import pytest
import torch

from dist_utils import run_distributed

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _need_gpus(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _close(a, b, k, tol=3e-2):
    scale = max(1.0, k ** 0.5)
    torch.testing.assert_close(a.float() / scale, b.float() / scale, rtol=tol, atol=tol)


def _worker(rank, world, nvls, ag_mode=None):
    import os

    import torch.distributed as dist

    if ag_mode is not None:      # the all-gather form (default: "gather" with nvls, else "pull")
        os.environ["SLAPO_B200_AG_MODE"] = ag_mode

    from slapo_b200.ops import native
    from slapo_b200.parallel import fused_tp as ft
    from slapo_b200.parallel.symm import SymmContext

    dev = torch.device("cuda", rank)
    # nvls: the reduction goes through the NVSwitch (multimem) instead of loading from every peer
    ctx = SymmContext(None, dev, nvls=nvls)
    torch.manual_seed(1234)
    ts, k, n = 256, 256, 384
    t = ts * world
    dt = torch.bfloat16
    # identical "global" tensors on every rank, each takes its slice
    x_full = torch.randn(t, k, device=dev, dtype=dt)
    w_col = torch.randn(world * n, k, device=dev, dtype=dt)      # column-parallel weight
    w_row = torch.randn(k, world * n, device=dev, dtype=dt)      # row-parallel weight [out, in]
    bias = torch.randn(k, device=dev, dtype=dt)
    g_col = torch.randn(t, world * n, device=dev, dtype=dt)
    g_row = torch.randn(t, k, device=dev, dtype=dt)

    # ---- column parallel with token-sharded input: ag_linear ----
    xs = x_full[rank * ts:(rank + 1) * ts].clone().requires_grad_(True)
    wl = w_col[rank * n:(rank + 1) * n].clone().requires_grad_(True)
    y = ft.ag_linear(xs, wl, None, ctx)
    y.backward(g_col[:, rank * n:(rank + 1) * n].contiguous())
    torch.cuda.synchronize()
    assert native.ops().device_status() == 0
    xf = x_full.float().requires_grad_(True)
    wf = w_col.float().requires_grad_(True)
    (xf @ wf.t()).backward(g_col.float())
    _close(y, (x_full.float() @ w_col.float().t())[:, rank * n:(rank + 1) * n], k)
    _close(xs.grad, xf.grad[rank * ts:(rank + 1) * ts], n * world)
    _close(wl.grad, wf.grad[rank * n:(rank + 1) * n], t)

    # ---- row parallel, reduce-scattered output: rs_linear ----
    h_full = torch.randn(t, world * n, device=dev, dtype=dt)
    hl = h_full[:, rank * n:(rank + 1) * n].clone().requires_grad_(True)
    wr = w_row[:, rank * n:(rank + 1) * n].clone().requires_grad_(True)
    b = bias.clone().requires_grad_(True)
    z = ft.rs_linear(hl, wr, b, ctx)
    z.backward(g_row[rank * ts:(rank + 1) * ts].contiguous())
    torch.cuda.synchronize()
    assert native.ops().device_status() == 0
    hf = h_full.float().requires_grad_(True)
    wrf = w_row.float().requires_grad_(True)
    ref = hf @ wrf.t() + bias.float()
    ref.backward(g_row.float())
    _close(z, ref[rank * ts:(rank + 1) * ts], n * world)
    _close(hl.grad, hf.grad[:, rank * n:(rank + 1) * n], k)
    _close(wr.grad, wrf.grad[:, rank * n:(rank + 1) * n], t)

    # ---- row parallel, all-reduced output: ar_linear ----
    hl2 = hl.detach().clone().requires_grad_(True)
    z2 = ft.ar_linear(hl2, wr.detach(), bias, ctx)
    torch.cuda.synchronize()
    assert native.ops().device_status() == 0
    _close(z2, ref.detach(), n * world)
    # several back-to-back operations reuse the buffers safely
    for _ in range(5):
        z3 = ft.ar_linear(hl2, wr.detach(), bias, ctx)
        y3 = ft.ag_linear(xs.detach(), wl.detach(), None, ctx)
    torch.cuda.synchronize()
    assert native.ops().device_status() == 0
    _close(z3, ref.detach(), n * world)
    _close(y3, (x_full.float() @ w_col.float().t())[:, rank * n:(rank + 1) * n], k)
    if ft.push_enabled(ctx):     # every staging slot went back to the pool
        assert not ft.stage_pool(ctx).out
    dist.barrier()


@pytest.mark.parametrize("nvls,ag_mode", [(False, None), (True, None), (False, "push"), (True, "push"),
                                          (False, "gather")])
@pytest.mark.parametrize("world", [2, 4])
def test_fused_tp_linears_on_peers(world, nvls, ag_mode):
    """nvls: reductions through the NVSwitch.  The all-gather is a multicast push kernel + pair
    GEMM with nvls and a fused pull without, unless ``ag_mode`` says otherwise (``push``: fused
    kernel with the owners' stores inside; without nvls the stores go rank by rank)."""
    _need_gpus(world)
    run_distributed(_worker, world, nvls, ag_mode, backend="nccl")


def _embed_worker(rank, world, sp_axis):
    import torch.distributed as dist

    from slapo_b200.ops import native
    from slapo_b200.ops.embedding import FusedVocabParallelEmbedding
    from slapo_b200.parallel.symm import SymmContext

    dev = torch.device("cuda", rank)
    ctx = SymmContext(None, dev, nvls=False)
    torch.manual_seed(21)
    vocab, hidden, b, s = 64 * world, 128, 4 * world, 16 * world
    table = torch.randn(vocab, hidden, device=dev).bfloat16()
    ids = torch.randint(0, vocab, (b, s), device=dev)
    g_full = torch.randn(b, s, hidden, device=dev).bfloat16()
    mod = FusedVocabParallelEmbedding(torch.nn.Parameter(table.chunk(world)[rank].clone()),
                                      rank * (vocab // world), ctx, sp_axis=sp_axis)
    for _ in range(2):   # twice: the output buffers alternate
        mod.weight.grad = None
        out = mod(ids)
        want = table[ids] if sp_axis is None else table[ids].chunk(world, dim=sp_axis)[rank]
        g = g_full if sp_axis is None else g_full.chunk(world, dim=sp_axis)[rank].contiguous()
        out.backward(g)
        torch.cuda.synchronize()
        assert native.ops().device_status() == 0
        assert torch.equal(out, want)
        ref = torch.zeros(vocab, hidden, device=dev)
        ref.index_add_(0, ids.reshape(-1), g_full.reshape(-1, hidden).float())
        torch.testing.assert_close(mod.weight.grad.float(), ref.chunk(world)[rank], rtol=2e-2,
                                   atol=2e-2)
    dist.barrier()


@pytest.mark.parametrize("sp_axis", [None, 0, 1])
def test_vocab_parallel_embedding_on_peers(sp_axis):
    _need_gpus(2)
    run_distributed(_embed_worker, 2, sp_axis, backend="nccl")
