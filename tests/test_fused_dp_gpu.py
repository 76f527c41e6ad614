"""Fused data-parallel kernels (gradient reduce-scatter by peer pulls, AdamW +
parameter all-gather by peer pushes).

Single GPU: the ranks are emulated one after the other over a
``LocalSymmContext`` with the peers' flags pre-set (two mutually waiting
kernels never run on one device).  Two GPUs: the engine with the fused path
against the same engine over NCCL."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _adamw_ref(w, g, m, v, decay, lr, b1, b2, eps, wd, step, coef):
    g = g * coef
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    bc1, bc2 = 1 - b1**step, 1 - b2**step
    upd = (m / bc1) / ((v / bc2).sqrt() + eps) + wd * w * decay
    return w - lr * upd, m, v


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_dp_emulated_ranks(world):
    from slapo_b200.ops import native
    from slapo_b200.parallel.fused_dp import FusedDP
    from slapo_b200.parallel.symm import LocalSymmContext

    torch.manual_seed(0)
    dev = torch.device("cuda")
    n_buckets, shard = 2, 8 * 1024 + 64          # two buckets, ragged grid tail
    per_bucket = shard * world
    total = n_buckets * per_bucket
    ctx = LocalSymmContext(world)
    fdps = [FusedDP(ctx.as_rank(r), total, torch.bfloat16, n_buckets, wait_seconds=0.05)
            for r in range(world)]
    grads = [torch.randn(total, device=dev).bfloat16() for _ in range(world)]
    params = torch.randn(total, device=dev).bfloat16()
    for r in range(world):
        fdps[r].flat_grad.copy_(grads[r])
        fdps[r].flat_param.copy_(params)
        fdps[r].flags.fill_(1)                    # every peer "ready" and "pushed" for step 1
    mean = torch.stack([g.float() for g in grads]).mean(0)
    dup = (torch.arange(shard, device=dev) % 3 == 0).to(torch.uint8)
    lr, betas, eps, wd = 1e-2, (0.9, 0.999), 1e-8, 0.01
    decay = torch.ones(shard, dtype=torch.uint8, device=dev)
    want_param = params.float().clone()
    state = {}
    for r in range(world):
        for b in range(n_buckets):
            lo = b * per_bucket + r * shard
            out = torch.empty(shard, device=dev, dtype=torch.bfloat16)
            fdps[r].grad_rs(b, 1, lo, out, dup, split=(b == 0))
            torch.testing.assert_close(out.float(), mean[lo:lo + shard], rtol=1e-2, atol=1e-2)
            state[(r, b)] = out
        parts = fdps[r].take_norm_parts()
        got = torch.cat([state[(r, b)] for b in range(n_buckets)]).float()
        mask = dup.bool().repeat(n_buckets)
        torch.testing.assert_close(parts[0], got[~mask].pow(2).sum(), rtol=1e-3, atol=1e-3)
        torch.testing.assert_close(parts[1], got[mask].pow(2).sum(), rtol=1e-3, atol=1e-3)
    coef = torch.tensor([0.5], device=dev)
    for r in range(world):
        for b in range(n_buckets):
            lo = b * per_bucket + r * shard
            g = state[(r, b)]
            master = params[lo:lo + shard].float().clone()
            m = torch.zeros(shard, device=dev)
            v = torch.zeros(shard, device=dev)
            w_ref, _, _ = _adamw_ref(master.clone(), g.float(), m.clone(), v.clone(), 1.0, lr,
                                     *betas, eps, wd, 1, 0.5)
            want_param[lo:lo + shard] = w_ref
            fdps[r].adamw_ag(1, b == n_buckets - 1, lo, g, master, m, v, decay, coef, lr, betas,
                             eps, wd, 1 - betas[0], 1 - betas[1])
            torch.testing.assert_close(master, w_ref, rtol=1e-5, atol=1e-6)
    torch.cuda.synchronize()
    assert native.ops().device_status() == 0
    for r in range(world):      # every rank's parameter buffer holds every slice
        torch.testing.assert_close(fdps[r].flat_param.float(), want_param, rtol=1e-2, atol=1e-2)


def test_fused_dp_wait_is_bounded():
    """A peer that never signals: the kernel gives up, sets the status word and returns."""
    from slapo_b200.ops import native
    from slapo_b200.parallel.fused_dp import FusedDP
    from slapo_b200.parallel.symm import LocalSymmContext

    ctx = LocalSymmContext(2)
    fdp = FusedDP(ctx.as_rank(0), 4096, torch.bfloat16, 1, wait_seconds=0.05)
    out = torch.zeros(2048, device="cuda", dtype=torch.bfloat16)
    native.ops().device_status()                  # clear
    fdp.grad_rs(0, 1, 0, out, None)               # nobody ever sets rank 1's flag
    torch.cuda.synchronize()
    assert native.ops().device_status() == 5
    assert native.ops().device_status() == 0      # reading clears it; the context is usable
    assert float(out.abs().sum()) == 0.0


def _dp_worker(rank, world):
    import copy

    import torch.distributed as dist

    from slapo_b200.ops import native
    from slapo_b200.parallel.mesh import DeviceMesh
    from slapo_b200.runtime.engine import TrainEngine

    dev = torch.device("cuda", rank)
    torch.manual_seed(0)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(512, 2048)
            self.b = torch.nn.Linear(2048, 512)
            self.n = torch.nn.LayerNorm(512)

        def forward(self, x, y):
            return {"loss": (self.n(self.b(torch.relu(self.a(x)))).float() - y).pow(2).mean()}

    base = Net().to(dev).bfloat16()
    mesh = DeviceMesh(pp=1, dp=world, tp=1)
    cfg = {"lr": 1e-2, "bucket_mb": 1.0, "clip_grad": 1.0}
    fused = TrainEngine(copy.deepcopy(base), dict(cfg), mesh=mesh)
    plain = TrainEngine(copy.deepcopy(base), dict(cfg, fused_dp=False), mesh=mesh)
    assert fused.fdp is not None and plain.fdp is None and len(fused.buckets) >= 2
    for step in range(4):
        g = torch.Generator(device="cpu").manual_seed(100 * step + rank)
        x = torch.randn(64, 512, generator=g).to(dev).bfloat16()
        y = torch.randn(64, 512, generator=g).to(dev)
        before = native.launch_count()
        l1 = fused.train_batch(x, y)
        assert native.launch_count() - before >= 3 * len(fused.buckets)
        l2 = plain.train_batch(x, y)
        torch.testing.assert_close(l1, l2, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(fused.last_grad_norm, plain.last_grad_norm, rtol=2e-2, atol=1e-3)
    assert native.ops().device_status() == 0
    torch.testing.assert_close(fused.flat_param.float(), plain.flat_param.float(), rtol=3e-2, atol=3e-2)
    # all ranks hold identical parameters after the pushes
    mine = fused.flat_param.float().clone()
    other = mine.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(mine, other)
    dist.barrier()


@pytest.mark.multigpu
def test_fused_dp_engine_two_gpus():
    from dist_utils import run_distributed

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_distributed(_dp_worker, 2, backend="nccl")


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("direction", ["RS->SR", "SR->RS"])
def test_fused_all_to_all_emulated_ranks(world, direction):
    """The reshard all-to-all as peer stores: every emulated rank pushes its blocks, then each
    rank's receive buffer must hold the resharded tensor."""
    from slapo_b200.ops import native
    from slapo_b200.parallel.fused_a2a import FusedAllToAll
    from slapo_b200.parallel.symm import LocalSymmContext

    torch.manual_seed(3)
    b, s, h = 3, 8 * world, 16 * world
    full = torch.randn(b, s, h, device="cuda").bfloat16()
    ctx = LocalSymmContext(world)
    a2as = [FusedAllToAll(ctx.as_rank(r), wait_seconds=0.05) for r in range(world)]
    if direction == "RS->SR":
        ins = [full.chunk(world, 2)[r].contiguous() for r in range(world)]
        want = [full.chunk(world, 1)[r] for r in range(world)]
        split_dim, cat_dim = -2, -1
    else:
        ins = [full.chunk(world, 1)[r].contiguous() for r in range(world)]
        want = [full.chunk(world, 2)[r] for r in range(world)]
        split_dim, cat_dim = -1, -2
    views = []
    for r in range(world):
        ctx.as_rank(r)
        ctx.epoch = 0                                   # SPMD: every rank counts the same epochs
        a2as[r].flag_buf.view(torch.int32, (8,)).fill_(1)   # the peers "sent" epoch 1 already
        assert a2as[r].supports(ins[r], split_dim, cat_dim, world)
        views.append(a2as[r].push(ins[r], split_dim, cat_dim))
    torch.cuda.synchronize()
    assert native.ops().device_status() == 0
    for r in range(world):
        assert torch.equal(views[r], want[r]), f"rank {r}"


def _a2a_worker(rank, world):
    import torch.distributed as dist

    from slapo_b200.ops import native
    from slapo_b200.parallel import reshard_ops
    from slapo_b200.parallel.symm import SymmContext

    dev = torch.device("cuda", rank)
    torch.manual_seed(5)
    full = torch.randn(2, 64, 256, device=dev).bfloat16()
    local = full.chunk(world, 2)[rank].contiguous().requires_grad_(True)
    ref = reshard_ops.reshard("RS->SR", local, None)            # NCCL all-to-all
    ref.backward(torch.ones_like(ref) * (rank + 1))
    g_ref = local.grad.clone()
    local.grad = None
    reshard_ops.enable_fused_all_to_all(None, SymmContext(None, device=dev))
    before = native.launch_count()
    out = reshard_ops.reshard("RS->SR", local, None)
    assert native.launch_count() == before + 1
    assert torch.equal(out, ref) and torch.equal(out, full.chunk(world, 1)[rank])
    out.backward(torch.ones_like(out) * (rank + 1))              # the backward is SR->RS, fused too
    assert torch.equal(local.grad, g_ref)
    assert native.ops().device_status() == 0
    dist.barrier()


@pytest.mark.multigpu
def test_fused_all_to_all_two_gpus():
    from dist_utils import run_distributed

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_distributed(_a2a_worker, 2, backend="nccl")


@pytest.mark.parametrize("world", [2, 4])
def test_vocab_parallel_embedding_emulated_ranks(world):
    """Every emulated rank stores the rows it owns into all ranks' outputs; afterwards each
    output equals the plain embedding lookup, and the backward gives each rank the gradient of
    its vocabulary slice."""
    from slapo_b200.ops import native
    from slapo_b200.ops.embedding import FusedVocabParallelEmbedding
    from slapo_b200.parallel.symm import LocalSymmContext

    torch.manual_seed(4)
    vocab, hidden = 64 * world, 256
    table = torch.randn(vocab, hidden, device="cuda").bfloat16()
    ids = torch.randint(0, vocab, (3, 50), device="cuda")
    ids[0, :4] = torch.tensor([0, vocab - 1, vocab // world, vocab // world - 1])   # shard edges
    want = table[ids]
    ctx = LocalSymmContext(world)
    mods = []
    for r in range(world):
        w = torch.nn.Parameter(table.chunk(world)[r].clone())
        mods.append(FusedVocabParallelEmbedding(w, r * (vocab // world), ctx.as_rank(r)))
    outs = []
    for r in range(world):
        ctx.as_rank(r)
        ctx.epoch = 0
        mods[r].flag_buf.view(torch.int32, (8,)).fill_(1)
        outs.append(mods[r](ids))           # a clone taken right after this rank's stores
    torch.cuda.synchronize()
    assert native.ops().device_status() == 0
    # the symmetric output of every rank is complete once all ranks have run
    for r in range(world):
        full = ctx.rank_view("vocab_embed_out_0", r, torch.bfloat16, (ids.numel(), hidden))
        assert torch.equal(full.view(3, 50, hidden), want), f"rank {r}"
    # backward: only the owned rows receive gradient
    g = torch.randn(3, 50, hidden, device="cuda").bfloat16()
    ref = torch.zeros(vocab, hidden, device="cuda")
    ref.index_add_(0, ids.reshape(-1), g.reshape(-1, hidden).float())
    for r in range(world):
        outs[r].backward(g)
        torch.testing.assert_close(mods[r].weight.grad.float(), ref.chunk(world)[r],
                                   rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("sp_axis", [0, 1])
@pytest.mark.parametrize("world", [2, 4])
def test_vocab_parallel_embedding_scatter_form_emulated_ranks(world, sp_axis):
    """Sequence-parallel form: the owner of a row stores it into the ONE rank that keeps the
    token; once all ranks have run, every rank's buffer holds exactly its chunk of the batch
    (axis 0) or of every sequence (axis 1)."""
    from slapo_b200.ops import native
    from slapo_b200.ops.embedding import FusedVocabParallelEmbedding
    from slapo_b200.parallel.symm import LocalSymmContext

    torch.manual_seed(5)
    vocab, hidden, b, s = 64 * world, 128, 8, 48
    table = torch.randn(vocab, hidden, device="cuda").bfloat16()
    ids = torch.randint(0, vocab, (b, s), device="cuda")
    want = table[ids].chunk(world, dim=sp_axis)
    ctx = LocalSymmContext(world)
    mods = [FusedVocabParallelEmbedding(torch.nn.Parameter(table.chunk(world)[r].clone()),
                                        r * (vocab // world), ctx.as_rank(r), sp_axis=sp_axis)
            for r in range(world)]
    with torch.no_grad():
        for r in range(world):
            ctx.as_rank(r)
            ctx.epoch = 0
            mods[r].flag_buf.view(torch.int32, (8,)).fill_(1)
            out = mods[r](ids)
            assert out.shape == want[r].shape
    torch.cuda.synchronize()
    assert native.ops().device_status() == 0
    for r in range(world):
        got = ctx.rank_view("vocab_embed_out_0", r, torch.bfloat16, tuple(want[r].shape))
        assert torch.equal(got, want[r]), f"rank {r}"
