"""Multi-GPU micro-benchmark of the fused compute + collective kernels.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m slapo_b200.bench.comm_bench

Times, on N GPUs of one node, the kernels that ``shard`` + ``sync`` lower to -
all-gather -> GEMM, GEMM -> reduce-scatter, GEMM -> all-reduce - on the
per-layer shapes of BERT-large under N-way tensor + sequence parallelism,
next to the unfused baseline (NCCL collective + cuBLAS GEMM), and the fused
data-parallel kernels against NCCL reduce-scatter / all-gather.  Every time
is device time (CUDA events), the maximum over ranks.  Each fused kernel is
reported as achieved / roofline, the roofline being the slower of FLOPs at
the measured GEMM peak and the bytes that must cross NVLink at the measured
peer-copy bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F

GEMM_PEAK_TFLOPS = 1645.7      # measured cuBLAS bf16 burst on this pool's B200
LINK_GBS = 770.0               # measured peer copy, per direction per GPU


def _time(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    torch.cuda.synchronize()
    us = torch.tensor([t0.elapsed_time(t1) * 1e3 / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(us, op=dist.ReduceOp.MAX)
    return float(us.item())


def _trace_summary(rank, name, scatter=False):
    """With SLAPO_B200_COMM_TRACE=1 the fused kernels record per-CTA time stamps; print, for the
    last launch, each phase's median / maximum over the CTAs in microseconds after the first
    CTA entered the kernel."""
    if os.environ.get("SLAPO_B200_COMM_TRACE") != "1" or rank != 0:
        return
    tr = torch.ops.slapo_b200.comm_trace()[:148].double()
    t0 = tr[:, 0].min()
    names = (["entry", "reduce_first", "reduce_last", "-", "-", "tiles_done", "exit"] if scatter
             else ["entry", "copy_first", "copy_last", "wait_begin", "wait_end", "tiles_done", "exit"])
    out = {}
    for i, nm in enumerate(names):
        if nm == "-":
            continue
        col = tr[:, i]
        col = col[col >= t0]
        if col.numel():
            rel = (col - t0) / 1e3
            out[nm] = [round(float(rel.median()), 1), round(float(rel.max()), 1)]
            if nm == "tiles_done":   # spread over the CTAs: deciles and the five slowest CTAs
                q = torch.quantile(rel, torch.linspace(0, 1, 11, dtype=rel.dtype))
                out["tiles_done_deciles"] = [round(float(v), 1) for v in q]
                out["slowest_ctas"] = [int(i) for i in torch.argsort(tr[:, i], descending=True)[:5]]
    w = tr[:, 7] / 1e3
    out["staged_wait_us"] = [round(float(w.median()), 1), round(float(w.max()), 1)]
    print(json.dumps({"trace": name, "median_max_us": out}), flush=True)


def _report(rank, name, us, flops, link_bytes, **extra):
    t_flops = flops / (GEMM_PEAK_TFLOPS * 1e12) * 1e6
    t_link = link_bytes / (LINK_GBS * 1e9) * 1e6
    roof = max(t_flops, t_link)
    if rank == 0:
        print(json.dumps({"kernel": name, "us": round(us, 1), "roofline_us": round(roof, 1),
                          "frac_roofline": round(roof / us, 3), "bound": "flops" if t_flops >= t_link
                          else "nvlink", "tflops": round(flops / us / 1e6, 1), **extra}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens-per-gpu", type=int, default=16384)   # 32 samples x 512
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--ffn", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ops", default="ag,rs,dp", help="comma list of ag, rs, dp")
    ap.add_argument("--no-baseline", action="store_true", help="skip the NCCL + cuBLAS lines")
    ap.add_argument("--nvls", type=int, default=-1,
                    help="1 / 0: reduce through the NVSwitch (multimem) or by peer loads; "
                         "-1: the context's default for the group size")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world, rank = dist.get_world_size(), dist.get_rank()
    from slapo_b200.ops import native
    from slapo_b200.parallel import fused_tp as ft
    from slapo_b200.parallel.symm import SymmContext

    ctx = SymmContext(None, nvls=None if args.nvls < 0 else bool(args.nvls))
    if rank == 0:
        print(json.dumps({"world": world, "nvls": ctx.nvls}), flush=True)
    dev, dt = torch.device("cuda", local), torch.bfloat16
    ts = args.tokens_per_gpu              # token shard of this rank (sequence parallel)
    t = ts * world                        # tokens seen by a TP region
    h, f = args.hidden, args.ffn
    torch.manual_seed(rank)
    ops = set(args.ops.split(","))
    for label, n_full, k in (("qkv", 3 * h, h), ("fc1", f, h)) if "ag" in ops else ():
        n = n_full // world
        x = torch.randn(ts, k, device=dev, dtype=dt)
        w = torch.randn(n, k, device=dev, dtype=dt)
        full = torch.empty(t, k, device=dev, dtype=dt)
        us = _time(lambda: ft.ag_gemm(ctx, x, w), args.iters)
        link = (world - 1) * ts * k * 2
        _report(rank, f"ag_gemm[{label}]", us, 2.0 * t * n * k, link, shape=[t, n, k], world=world)
        _trace_summary(rank, f"ag_gemm[{label}]")

        dist.all_gather_into_tensor(full, x)
        ref = F.linear(full, w)
        # owner-pushed forms: "push" inside the GEMM kernel, "gather" = push kernel + pair GEMM
        for mode in ("push", "gather"):
            us = _time(lambda: ft.ag_gemm_pushed(ctx, x, w, mode=mode)[0], args.iters)
            y_push, gathered, token = ft.ag_gemm_pushed(ctx, x, w, keep=True, mode=mode)
            err = float((y_push.float() - ref.float()).abs().max() / ref.float().abs().max())
            same = bool(torch.equal(gathered, full))
            ft.stage_pool(ctx).release(token)
            _report(rank, f"ag_gemm_{mode}[{label}]", us, 2.0 * t * n * k, link, shape=[t, n, k],
                    world=world, max_rel_err=round(err, 5), gathered_equal=same)
            if mode == "push":
                _trace_summary(rank, f"ag_gemm_push[{label}]")

        def base():
            dist.all_gather_into_tensor(full, x)
            return F.linear(full, w)

        if not args.no_baseline:
            us_b = _time(base, args.iters)
            _report(rank, f"nccl_all_gather+cublas[{label}]", us_b, 2.0 * t * n * k, link,
                    shape=[t, n, k], world=world)
    for label, n, k_full in (("attn_out", h, h), ("fc2", h, f)) if "rs" in ops else ():
        k = k_full // world
        x = torch.randn(t, k, device=dev, dtype=dt)
        w = torch.randn(n, k, device=dev, dtype=dt)
        out = torch.empty(ts, n, device=dev, dtype=dt)
        link = (world - 1) * ts * n * 2
        us = _time(lambda: ft.gemm_rs(ctx, x, w), args.iters)
        _report(rank, f"gemm_rs[{label}]", us, 2.0 * t * n * k, link, shape=[t, n, k], world=world)
        _trace_summary(rank, f"gemm_rs[{label}]", scatter=True)

        def base_rs():
            dist.reduce_scatter_tensor(out, F.linear(x, w))
            return out

        if not args.no_baseline:
            us_b = _time(base_rs, args.iters)
            _report(rank, f"cublas+nccl_reduce_scatter[{label}]", us_b, 2.0 * t * n * k, link,
                    shape=[t, n, k], world=world)
        us = _time(lambda: ft.gemm_ar(ctx, x, w), args.iters)
        _report(rank, f"gemm_ar[{label}]", us, 2.0 * t * n * k, 2 * link, shape=[t, n, k],
                world=world)
    # fused data parallel: one 64 MiB bucket
    if "dp" in ops:
        from slapo_b200.parallel.fused_dp import FusedDP

        elems = 32 * 2**20
        fdp = FusedDP(ctx, elems, dt, 1)
        shard = elems // world
        out = torch.empty(shard, device=dev, dtype=dt)
        state = {"epoch": 0}

        def rs():
            state["epoch"] += 1
            fdp.grad_rs(0, state["epoch"], rank * shard, out, None)

        us = _time(rs, args.iters)
        _report(rank, "dp_grad_rs[64MiB]", us, 0.0, (world - 1) * shard * 2, world=world)
        grad = torch.randn(elems, device=dev, dtype=dt)
        us = _time(lambda: dist.reduce_scatter_tensor(out, grad, op=dist.ReduceOp.AVG), args.iters)
        _report(rank, "nccl_reduce_scatter[64MiB]", us, 0.0, (world - 1) * shard * 2, world=world)
    if rank == 0:
        print(json.dumps({"device_status": int(native.ops().device_status())}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
