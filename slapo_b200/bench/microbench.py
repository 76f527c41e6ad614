"""Micro-benchmarks of the hand-written kernels against their rooflines.

    python -m slapo_b200.bench.microbench --op all            # full-size shapes
    python -m slapo_b200.bench.microbench --op ln --small     # small case for profilers

Every number is CUDA-event timed on the launching stream after warm-up, on
inputs larger than the 126 MB L2 unless ``--small`` is given.  Prints one JSON
line per measurement: achieved GB/s or TFLOP/s and, when the measured peaks
file is present, the fraction of the measured peak.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import functional as NF
from ..ops import native
from ..ops.flash_attn import flash_attention_qkvpacked


def _peaks():
    path = os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, iters=20, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / iters * 1e3  # microseconds


def report(name, us, nbytes=None, flops=None, **extra):
    hbm, tf, kind = _peaks()
    rec = {"kernel": name, "us": round(us, 1)}
    if nbytes is not None:
        gbs = nbytes / us / 1e3
        rec.update(gbs=round(gbs, 1), frac_hbm=round(gbs / hbm, 3))
    if flops is not None:
        t = flops / us / 1e6
        rec.update(tflops=round(t, 1), frac_bf16=round(t / tf, 3))
    rec["peaks"] = kind
    rec.update(extra)
    print(json.dumps(rec), flush=True)


def bench_ln(small, iters):
    rows, cols = (32768, 1024) if small else (65536, 1024)   # several tensors of 64 MB: beyond L2
    dt = torch.bfloat16
    x = torch.randn(rows, cols, device="cuda", dtype=dt, requires_grad=True)
    r = torch.randn_like(x)
    w = torch.ones(cols, device="cuda", dtype=dt, requires_grad=True)
    b = torch.zeros(cols, device="cuda", dtype=dt, requires_grad=True)
    elt = rows * cols * 2

    def fwd():
        return NF.dropout_add_layer_norm(x, b, r, w, b, 0.1, 1e-12, True)[0]

    y = fwd()
    g = torch.randn_like(y)
    t_f = timeit(fwd, iters)
    report("dropout_add_ln_fwd", t_f, nbytes=4 * elt, rows=rows, cols=cols)

    def both():
        fwd().backward(g)

    t_b = timeit(both, iters) - t_f
    report("dropout_add_ln_bwd", t_b, nbytes=4 * elt, rows=rows, cols=cols)


def bench_gelu(small, iters):
    rows, cols = (4096, 4096) if small else (32768, 4096)
    dt = torch.bfloat16
    x = torch.randn(rows, cols, device="cuda", dtype=dt, requires_grad=True)
    b = torch.zeros(cols, device="cuda", dtype=dt, requires_grad=True)
    elt = rows * cols * 2
    t_f = timeit(lambda: NF.bias_act(x, b, "gelu"), iters)
    report("bias_gelu_fwd", t_f, nbytes=2 * elt, rows=rows, cols=cols)
    g = torch.randn(rows, cols, device="cuda", dtype=dt)

    def both():
        NF.bias_act(x, b, "gelu").backward(g)

    report("bias_gelu_bwd", timeit(both, iters) - t_f, nbytes=3 * elt, rows=rows, cols=cols)


def bench_attn(small, iters):
    shapes = [(64, 512, 16, 64, False)] if small else [
        (32, 512, 16, 64, False), (4, 1024, 20, 128, True), (8, 2048, 16, 64, True)]
    for (bsz, s, h, d, causal) in shapes:
        qkv = torch.randn(bsz, s, h, 3, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        flops = 4 * bsz * h * s * s * d * (0.5 if causal else 1.0)
        for p in (0.0, 0.1):
            out = flash_attention_qkvpacked(qkv, causal=causal, p=p)
            g = torch.randn_like(out)
            t_f = timeit(lambda: flash_attention_qkvpacked(qkv, causal=causal, p=p), iters)
            report("flash_fwd", t_f, flops=flops, shape=[bsz, s, h, d], causal=causal, p=p)

            def both():
                flash_attention_qkvpacked(qkv, causal=causal, p=p).backward(g)

            report("flash_bwd", timeit(both, iters) - t_f, flops=2.5 * flops,
                   shape=[bsz, s, h, d], causal=causal, p=p)


def bench_gemm(small, iters):
    shapes = [(8192, 8192, 2048)] if small else [
        (16384, 4096, 1024), (16384, 1024, 4096), (16384, 3072, 1024), (8192, 8192, 8192)]
    for (m, n, k) in shapes:
        a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        ops = native.ops()
        t0 = timeit(lambda: ops.gemm_out(a, b, None, -1, False, False, out, None, 2, False), iters)
        t1 = timeit(lambda: ops.gemm_out(a, b, None, -1, False, False, out, None, 1, False), iters)
        t2 = timeit(lambda: torch.matmul(a, b.t(), out=out), iters)
        report("gemm2_tc05 (CTA pairs)", t0, flops=2 * m * n * k, shape=[m, n, k])
        report("gemm_tc05 (single CTA)", t1, flops=2 * m * n * k, shape=[m, n, k])
        report("gemm_cublas", t2, flops=2 * m * n * k, shape=[m, n, k])


def bench_comm(small, iters):
    """Fused GEMM + collective kernels as ONE emulated rank of a 2-rank group whose "peer"
    buffers live on this GPU too, with the peer's flags pre-set: the kernel runs its full
    code path (copier warps, staging, pull-based reduction) and its tensor-core / memory
    behaviour can be profiled on a single GPU; NVLink time is not part of these numbers."""
    from slapo_b200.parallel import fused_tp as ft
    from slapo_b200.parallel.symm import LocalSymmContext

    world = 2
    ts, k, n = (4096, 1024, 4096) if small else (8192, 1024, 4096)
    ctx = LocalSymmContext(world, wait_seconds=0.05)
    shards = [torch.randn(ts, k, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    for r in range(world):
        buf = ctx.as_rank(r).buffer("ag_in", ts * k * 2)
        buf.view(torch.bfloat16, (ts, k)).copy_(shards[r])
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    ctx.as_rank(0)

    def ag():
        ctx.preset_flags(ctx.epoch + 1)
        return ft.ag_gemm(ctx, shards[0], w, None, staged=ctx.buffer("ag_in", ts * k * 2))

    report("ag_gemm_emulated", timeit(ag, iters), flops=2 * ts * world * n * k,
           shape=[ts * world, n, k], world=world)
    # pushed form: this rank stores its rows into both slots; the peer's rows and block flags
    # are put into this rank's slot beforehand (once: flags only have to be >= the epoch)
    nbytes = ts * world * k * 2
    slot = ctx.buffer(f"ag_slot_{nbytes}_0", ft.RECV_HEADER_BYTES + nbytes)
    ctx.as_rank(1).buffer(f"ag_slot_{nbytes}_0", ft.RECV_HEADER_BYTES + nbytes)
    ctx.as_rank(0)
    slot.view(torch.bfloat16, (ts * world, k), ft.RECV_HEADER_BYTES).copy_(torch.cat(shards, 0))
    slot.view(torch.int32, (ts * world // 128 * 16,))[ts // 128 * 16:] = 1 << 30   # 16 flags per block

    def ag_push():
        ctx.preset_flags(ctx.epoch + 1)
        return ft.ag_gemm_pushed(ctx, shards[0], w)[0]

    report("ag_gemm_push_emulated", timeit(ag_push, iters), flops=2 * ts * world * n * k,
           shape=[ts * world, n, k], world=world)
    x = torch.randn(ts * world, n, device="cuda", dtype=torch.bfloat16)
    w2 = torch.randn(k, n, device="cuda", dtype=torch.bfloat16)

    ctx.buffer("rs_recv", ft.RECV_HEADER_BYTES + ts * world * k * 2)

    def rs():
        ctx.preset_flags(ctx.epoch + 1, ready=True, done=True, done2=True)
        ctx.preset_block_flags("rs_recv", ctx.epoch + 1, ts // 128)
        return ft.gemm_rs(ctx, x, w2, None)

    report("gemm_rs_emulated", timeit(rs, iters), flops=2 * ts * world * n * k,
           shape=[ts * world, k, n], world=world)


def bench_peer(small, iters):
    """The other peer-memory kernels as ONE emulated rank of a 4-rank group on this GPU (peer
    buffers are local memory, the peers' flags are preset): data-parallel gradient
    reduce-scatter, AdamW + parameter all-gather, the reshard all-to-all, the vocabulary-
    parallel embedding (both forms), the plain peer gather and the GEMM -> all-reduce.  Every
    kernel runs its full code path; no byte crosses NVLink, so the figures describe the memory
    side only (the real-NVLink times come from `comm_bench` on several GPUs)."""
    from slapo_b200.ops.embedding import FusedVocabParallelEmbedding
    from slapo_b200.parallel import fused_tp as ft
    from slapo_b200.parallel.fused_a2a import FusedAllToAll
    from slapo_b200.parallel.fused_dp import FusedDP
    from slapo_b200.parallel.symm import LocalSymmContext

    world, dev, dt = 4, torch.device("cuda"), torch.bfloat16
    ctx = LocalSymmContext(world, wait_seconds=0.05)
    # ---- data parallel: one bucket of 64 MiB (16 MiB for captures)
    elems = (8 if small else 32) * 2**20
    shard = elems // world
    fdps = [FusedDP(ctx.as_rank(r), elems, dt, 1, wait_seconds=0.05) for r in range(world)]
    for f in fdps:
        f.flat_grad.normal_()
        f.flat_param.normal_()
    out = torch.empty(shard, device=dev, dtype=dt)
    state = {"epoch": 0}

    def rs():
        state["epoch"] += 1
        for f in fdps:
            f.flags.fill_(state["epoch"])
        fdps[0].grad_rs(0, state["epoch"], 0, out, None)

    report("dp_grad_rs_emulated", timeit(rs, iters), nbytes=(world + 1) * shard * 2,
           elems=elems, world=world)
    master = torch.randn(shard, device=dev)
    m, v = torch.zeros(shard, device=dev), torch.zeros(shard, device=dev)
    decay = torch.ones(shard, dtype=torch.uint8, device=dev)
    coef = torch.ones(1, device=dev)

    def ag():
        state["epoch"] += 1
        for f in fdps:
            f.flags.fill_(state["epoch"])
        fdps[0].adamw_ag(state["epoch"], True, 0, out, master, m, v, decay, coef, 1e-4, (0.9, 0.999),
                         1e-8, 0.01, 0.1, 0.001)

    report("dp_adamw_ag_emulated", timeit(ag, iters),
           nbytes=shard * (2 + 3 * 8 + 1) + world * shard * 2, elems=elems, world=world)
    # ---- reshard all-to-all: [B, S, H / world] -> [B, S / world, H]
    b, s_len, h = (8, 512, 1024) if small else (32, 512, 1024)
    inp = torch.randn(b, s_len, h // world, device=dev, dtype=dt)
    a2a = FusedAllToAll(ctx.as_rank(0), wait_seconds=0.05)

    def a2a_fn():
        a2a.flag_buf.view(torch.int32, (8,)).fill_(ctx.epoch + 1)
        return a2a.push(inp, -2, -1)

    report("peer_all_to_all_emulated", timeit(a2a_fn, iters), nbytes=2 * inp.numel() * 2,
           shape=list(inp.shape), world=world)
    # ---- vocabulary-parallel embedding, all-gather and scatter forms
    vocab, hidden = 30528, 1024
    ids = torch.randint(0, vocab // world, (b, s_len), device=dev)   # every row owned by rank 0
    for sp_axis, label in ((None, "all_gather"), (0, "scatter")):
        emb = FusedVocabParallelEmbedding(
            torch.nn.Parameter(torch.randn(vocab // world, hidden, device=dev, dtype=dt)), 0,
            ctx.as_rank(0), sp_axis=sp_axis)

        def embed():
            emb.flag_buf.view(torch.int32, (8,)).fill_(ctx.epoch + 1)
            with torch.no_grad():
                return emb(ids)

        stores = world if sp_axis is None else 1
        report(f"vocab_embed_fwd_emulated[{label}]", timeit(embed, iters),
               nbytes=ids.numel() * hidden * 2 * (1 + stores), tokens=ids.numel(), world=world)
    # ---- plain peer gather of a [ts, k] shard
    ts, k = (2048, 1024) if small else (8192, 1024)
    shard_t = torch.randn(ts, k, device=dev, dtype=dt)

    def gather():
        ctx.preset_flags(ctx.epoch + 1)
        return ft.peer_gather(ctx, shard_t, "gather_bench")

    report("peer_gather_emulated", timeit(gather, iters), nbytes=2 * world * ts * k * 2,
           shape=[world * ts, k], world=world)
    # ---- GEMM -> all-reduce
    n = 1024
    x = torch.randn(ts * world, k, device=dev, dtype=dt)
    w = torch.randn(n, k, device=dev, dtype=dt)
    ctx.buffer("ar_recv", ft.RECV_HEADER_BYTES + ts * world * n * 2)

    def ar():
        ctx.preset_flags(ctx.epoch + 1, ready=True, done=True, done2=True)
        ctx.preset_block_flags("ar_recv", ctx.epoch + 1, ts // 128)
        return ft.gemm_ar(ctx, x, w, None)

    report("gemm_ar_emulated", timeit(ar, iters), flops=2 * ts * world * n * k,
           shape=[ts * world, n, k], world=world)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all",
                    choices=["all", "ln", "gelu", "attn", "gemm", "comm", "peer"])
    ap.add_argument("--small", action="store_true", help="small inputs for profiler captures")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    assert native.available(), native.load_error()
    todo = ["ln", "gelu", "attn", "gemm"] if args.op == "all" else [args.op]
    for op in todo:
        {"ln": bench_ln, "gelu": bench_gelu, "attn": bench_attn, "gemm": bench_gemm,
         "comm": bench_comm, "peer": bench_peer}[op](
            args.small, args.iters)
    print(json.dumps({"device_status": int(native.ops().device_status())}))


if __name__ == "__main__":
    main()
