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
import torch.nn.functional as F

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
    rows, cols = (4096, 1024) if small else (65536, 1024)
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
        t1 = timeit(lambda: native.ops().gemm(a, b, None, -1, False, False), iters)
        t2 = timeit(lambda: F.linear(a, b), iters)
        report("gemm_tc05", t1, flops=2 * m * n * k, shape=[m, n, k])
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
    x = torch.randn(ts * world, n, device="cuda", dtype=torch.bfloat16)
    w2 = torch.randn(k, n, device="cuda", dtype=torch.bfloat16)

    ctx.buffer("rs_recv", ft.RECV_HEADER_BYTES + ts * world * k * 2)

    def rs():
        ctx.preset_flags(ctx.epoch + 1, ready=True, done=True, done2=True)
        ctx.preset_block_flags("rs_recv", ctx.epoch + 1, ts // 128)
        return ft.gemm_rs(ctx, x, w2, None)

    report("gemm_rs_emulated", timeit(rs, iters), flops=2 * ts * world * n * k,
           shape=[ts * world, k, n], world=world)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all", choices=["all", "ln", "gelu", "attn", "gemm", "comm"])
    ap.add_argument("--small", action="store_true", help="small inputs for profiler captures")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    assert native.available(), native.load_error()
    todo = ["ln", "gelu", "attn", "gemm"] if args.op == "all" else [args.op]
    for op in todo:
        {"ln": bench_ln, "gelu": bench_gelu, "attn": bench_attn, "gemm": bench_gemm,
         "comm": bench_comm}[op](
            args.small, args.iters)
    print(json.dumps({"device_status": int(native.ops().device_status())}))


if __name__ == "__main__":
    main()
