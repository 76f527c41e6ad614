"""General training / benchmark entry for every model of the zoo.

    python -m slapo_b200.bench.train --model opt-2.7b --tp 4 --pp 2 --batch-size 4 \
        --micro-batches 16 --seq-len 1024 --steps 10

Launch under ``torchrun`` for more than one rank (one process per GPU; on a
machine without GPUs the same command runs on CPU ranks with gloo, which is
what the tests do with tiny configurations).  ``world = pp * dp * tp``; ``dp``
defaults to what is left after ``--tp`` and ``--pp``.  The script applies the
model's scheduling recipe, builds the native engine (ZeRO-1 data parallelism,
fused tensor-parallel kernels, 1F1B pipeline), trains on synthetic data of
the benchmark shape and prints one JSON record per run on rank 0:

    {"model": ..., "samples_per_sec": ..., "ms_per_step": ..., "max_mem_mb": ...,
     "param_per_gpu_m": ..., "tp": ..., "pp": ..., "dp": ..., "batch_size": ..., ...}

which is the format the auto-tuner's ``native`` log parser reads.  It plays
the role of the reference's per-model ``examples/*/deepspeed_hf.py`` and
``megatron_hf.py`` scripts (examples/bert/deepspeed_hf.py:1-260 of the
reference) with one engine instead of two external runtimes.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def parse_args(argv=None):
    ap = argparse.ArgumentParser("slapo_b200 training benchmark")
    ap.add_argument("--model", default="bert-large")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=0, help="0 = world / (tp * pp)")
    ap.add_argument("--batch-size", type=int, default=8,
                    help="samples per micro-batch per data-parallel replica")
    ap.add_argument("--micro-batches", type=int, default=1,
                    help="micro-batches per step (pipeline depth fill / gradient accumulation)")
    ap.add_argument("--seq-len", type=int, default=0)
    ap.add_argument("--seq-len-dec", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="override the depth (smoke runs)")
    ap.add_argument("--hidden", type=int, default=0, help="override the width (smoke runs)")
    ap.add_argument("--heads", type=int, default=0, help="override the head count (smoke runs)")
    ap.add_argument("--vocab", type=int, default=0, help="override the vocabulary (smoke runs)")
    ap.add_argument("--ckpt-ratio", type=float, default=0.0)
    ap.add_argument("--sequence-parallel", action="store_true")
    ap.add_argument("--no-fuse", action="store_true")
    ap.add_argument("--attn-op", default="auto")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--seed", type=int, default=2013)
    ap.add_argument("--save", default=None, help="write a sharded checkpoint here at the end")
    ap.add_argument("--resume", default=None, help="resume from this sharded checkpoint")
    ap.add_argument("--log-file", default=None, help="also append the JSON record to this file")
    ap.add_argument("--hang-dump", type=float, default=0.0,
                    help="dump every thread's Python stack to stderr after this many seconds "
                         "(and every such interval again): shows where a stuck rank waits")
    ap.add_argument("--no-fused-dp", action="store_true",
                    help="data parallelism through NCCL instead of the peer-memory kernels")
    ap.add_argument("--p2p-mode", default=None, choices=["paired", "overlap"],
                    help="pipeline transfers: one batched send + receive group per neighbour, "
                         "waited for (default next to the fused tensor-parallel kernels), or "
                         "side-stream transfers posted ahead (default otherwise)")
    ap.add_argument("--profile-table", default=None,
                    help="after the timed steps run two more under torch.profiler and write, per "
                         "rank, PATH.rank<r>.txt: the top device kernels and how much of the "
                         "send / receive kernels' time ran concurrently with other kernels")
    return ap.parse_args(argv)


def profile_overlap(step_fn, path, rank, steps=2):
    """Kernel table of ``steps`` steps and the overlap of point-to-point transfers with compute.

    The overlap is computed from the device-side intervals of the profiler's kernel events:
    the time covered by NCCL send / receive kernels, and the part of it during which at least
    one other kernel was running on the same device.  (Times taken under a profiler are not
    benchmark numbers; the table shows structure.)"""
    import torch
    from torch.autograd import DeviceType
    from torch.profiler import ProfilerActivity, profile

    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    with profile(activities=acts) as prof:
        for _ in range(steps):
            step_fn()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
    kernels = [e for e in prof.events() if e.device_type == DeviceType.CUDA and e.time_range is not None]
    p2p = [(e.time_range.start, e.time_range.end) for e in kernels
           if "SendRecv" in e.name or "sendrecv" in e.name.lower()]
    other = sorted((e.time_range.start, e.time_range.end) for e in kernels
                   if "nccl" not in e.name.lower() and "Memcpy" not in e.name and "Memset" not in e.name)
    merged = []
    for a, b in other:                       # union of the compute intervals
        if merged and a <= merged[-1][1]:
            merged[-1][1] = max(merged[-1][1], b)
        else:
            merged.append([a, b])
    total = sum(b - a for a, b in p2p)
    covered = 0.0
    for a, b in p2p:
        for c, d in merged:
            if d <= a:
                continue
            if c >= b:
                break
            covered += min(b, d) - max(a, c)
    sort_key = "cuda_time_total" if torch.cuda.is_available() else "cpu_time_total"
    table = prof.key_averages().table(sort_by=sort_key, row_limit=14, max_name_column_width=60)
    with open(f"{path}.rank{rank}.txt", "w", encoding="utf-8") as fh:
        fh.write(f"rank {rank}: {len(p2p)} send/receive kernels in {steps} steps, {total / 1e3:.2f} ms in "
                 f"total, {covered / 1e3:.2f} ms of it ({100.0 * covered / max(total, 1e-9):.0f} %) while "
                 "another kernel of this rank was running\n\n")
        fh.write(table)
    return {"p2p_kernels": len(p2p), "p2p_ms": total / 1e3, "p2p_overlapped_ms": covered / 1e3}


def _even_cuts(n_layers, n_stages):
    from slapo_b200.parallel.mesh import generate_pipeline_cuts

    return generate_pipeline_cuts(n_layers, n_stages)


def setup_distributed():
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if use_cuda:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo")
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    return world, rank, device


def build_engine(args, world, device):
    import torch

    import slapo_b200 as slapo
    from slapo_b200.models.zoo import get_model_spec
    from slapo_b200.parallel.mesh import DeviceMesh

    tp, pp = args.tp, args.pp
    dp = args.dp or world // (tp * pp)
    if tp * pp * dp != world:
        raise ValueError(f"tp {tp} x pp {pp} x dp {dp} != world size {world}")
    mesh = DeviceMesh(pp=pp, dp=dp, tp=tp) if world > 1 else None
    import dataclasses

    spec = get_model_spec(args.model)
    cfg = spec.config
    if not isinstance(cfg, dict):
        fields = {f.name for f in dataclasses.fields(cfg)}
        if args.layers:
            for key in ("num_hidden_layers", "num_layers", "num_decoder_layers"):
                if key in fields:
                    setattr(cfg, key, args.layers)
            spec.num_layers = args.layers
        if args.hidden:
            for key in ("hidden_size", "d_model"):
                if key in fields:
                    setattr(cfg, key, args.hidden)
            for key, mult in (("intermediate_size", 4), ("ffn_dim", 4), ("d_ff", 4)):
                if key in fields:
                    setattr(cfg, key, mult * args.hidden)
        if args.heads:
            for key in ("num_attention_heads", "num_heads"):
                if key in fields:
                    setattr(cfg, key, args.heads)
            if "d_kv" in fields:
                cfg.d_kv = cfg.d_model // args.heads
        if args.vocab and "vocab_size" in fields:
            cfg.vocab_size = args.vocab
        seq = args.seq_len or spec.default_seq
        for key in ("max_position_embeddings", "n_positions"):
            if key in fields and getattr(cfg, key) < seq:
                setattr(cfg, key, seq)
    sp = args.sequence_parallel and tp > 1
    slapo.set_random_seed(args.seed, dp_rank=mesh.dp_rank if mesh else 0,
                          pp_rank=mesh.pp_rank if mesh else 0,
                          tp_rank=mesh.tp_rank if mesh else 0, always_enable_tp_seed=sp)
    on_gpu = device.type == "cuda"
    if on_gpu:
        with slapo.init_empty_weights():
            model = spec.build()
    else:
        model = spec.build()
        if hasattr(model, "init_weights"):
            model.init_weights()
    kwargs = dict(model_config=cfg, group=mesh.schedule_group if mesh else None,
                  ckpt_ratio=args.ckpt_ratio, fuse=not args.no_fuse, attn_op_name=args.attn_op,
                  bf16=args.dtype == "bf16", fp16=args.dtype == "fp16")
    if spec.schedule_key in ("bert", "roberta", "gpt2", "gpt_neo", "opt"):
        kwargs["sequence_parallel"] = sp
        # token shards along the batch axis: gathered rows are a plain concatenation, which
        # is what the fused all-gather -> GEMM kernel consumes
        kwargs["sequence_parallel_axis"] = 0
    if pp > 1:
        if spec.kind == "seq2seq":
            half = pp // 2
            kwargs["pipeline_cuts"] = [_even_cuts(spec.num_layers, half),
                                       _even_cuts(spec.num_layers, pp - half)]
        elif spec.kind == "image":
            depths = cfg["block_size"][1]
            cuts = [[] for _ in depths]
            total, per = sum(depths), sum(depths) / pp
            acc, want = 0, 1
            for gi, d in enumerate(depths):
                for bi in range(d):
                    acc += 1
                    if want < pp and acc >= per * want and acc < total:
                        cuts[gi].append(bi)
                        want += 1
            kwargs["pipeline_cuts"] = cuts
        else:
            kwargs["pipeline_cuts"] = _even_cuts(spec.num_layers, pp)
    sch = slapo.model_schedule.apply_schedule(model, spec.schedule_key, **kwargs)
    tp_group = mesh.tp_group if mesh else None
    vocab_parallel = tp > 1 and spec.kind != "image"
    loss_fn = spec.loss_fn(tp_group, vocab_parallel)
    build_kwargs = dict(target="native", mesh=mesh, loss_fn=loss_fn,
                        config={"lr": args.lr, "weight_decay": 0.01, "clip_grad": 1.0,
                                "fused_dp": not args.no_fused_dp,
                                "grad_accum_steps": args.micro_batches if pp == 1 else 1})
    if pp > 1:
        build_kwargs["num_micro_batches"] = args.micro_batches
        if getattr(args, "p2p_mode", None):
            build_kwargs["config"]["p2p_mode"] = args.p2p_mode
    if not on_gpu:
        build_kwargs["init_weights"] = False
    elif hasattr(model, "_init_weights"):
        # the model's own initialiser also after pipeline partitioning (the split graph
        # module has lost the method, and PyTorch's per-layer defaults are another scheme)
        build_kwargs["init_weights"] = model._init_weights
    engine, _ = slapo.build(sch, **build_kwargs)
    return engine, spec, mesh, dp


def run(args):
    import torch
    import torch.distributed as dist

    from slapo_b200 import ckpt
    from slapo_b200.runtime.engine import StepTimer

    world, rank, device = setup_distributed()
    engine, spec, mesh, dp = build_engine(args, world, device)
    pp = args.pp
    inner = getattr(engine, "inner", engine)
    start_step = 0
    if args.resume:
        info = ckpt.load_checkpoint(args.resume, inner.model, inner, mesh=mesh)
        start_step = info["step"]
    dp_rank = mesh.dp_rank if mesh else 0
    # pipeline engines take the whole step's samples and split them; the plain engine is
    # called once per micro-batch (gradient accumulation)
    per_call = args.batch_size * (args.micro_batches if pp > 1 else 1)
    calls = 1 if pp > 1 else args.micro_batches
    seq = args.seq_len or spec.default_seq
    seq_dec = args.seq_len_dec or spec.default_seq_dec
    batches = [spec.make_batch(per_call, seq, seq_dec, seed=args.seed + 17 * dp_rank + i,
                               device=device) for i in range(calls)]
    if spec.kind == "image":   # images follow the parameter dtype
        pdtype = next(inner.model.parameters()).dtype
        batches = [(tuple(t.to(pdtype) for t in inputs), labels) for inputs, labels in batches]

    def step():
        loss = None
        for inputs, labels in batches:
            loss = engine.train_batch(*inputs, labels=labels)
        return loss

    loss = None
    for _ in range(args.warmup):
        loss = step()
    timer = StepTimer(device)
    if world > 1:
        dist.barrier()
    timer.start()
    for _ in range(args.steps):
        loss = step()
    ms = timer.stop()
    if world > 1:
        dist.barrier()
        ms = StepTimer.max_over_ranks(ms, device)
    samples = args.batch_size * args.micro_batches * dp * args.steps
    n_params = sum(p.numel() for p in inner.model.parameters())
    record = {
        "model": args.model, "samples_per_sec": samples / (ms / 1e3) if ms > 0 else 0.0,
        "ms_per_step": ms / max(args.steps, 1), "steps": args.steps, "warmup": args.warmup,
        "tp": args.tp, "pp": pp, "dp": dp, "batch_size": args.batch_size,
        "micro_batches": args.micro_batches, "seq_len": seq, "ckpt_ratio": args.ckpt_ratio,
        "sequence_parallel": bool(args.sequence_parallel and args.tp > 1), "dtype": args.dtype,
        "param_per_gpu_m": n_params / 1e6, "start_step": start_step,
        "max_mem_mb": (torch.cuda.max_memory_allocated() / 2**20) if device.type == "cuda" else 0.0,
        "loss": float(loss) if loss is not None and torch.is_tensor(loss) and loss.numel() == 1 else None,
        "device": device.type, "data": "synthetic",
    }
    if args.save:
        ckpt.save_checkpoint(args.save, inner.model, inner, mesh=mesh)
    if args.profile_table and device.type == "cuda":
        record["p2p_overlap"] = profile_overlap(step, args.profile_table, rank)
    if rank == 0:
        line = json.dumps(record)
        print(line, flush=True)
        if args.log_file:
            with open(args.log_file, "a", encoding="utf-8") as fh:
                fh.write(line + "\n")
    if world > 1:
        dist.destroy_process_group()
    return record


def main(argv=None):
    args = parse_args(argv)
    if args.hang_dump > 0:
        import faulthandler

        faulthandler.dump_traceback_later(args.hang_dump, repeat=True, file=sys.stderr)
    t0 = time.time()
    try:
        run(args)
    except Exception as err:  # the tuner classifies failures from the log text
        import torch

        if isinstance(err, torch.OutOfMemoryError):
            print("torch.OutOfMemoryError: CUDA out of memory.", flush=True)
        raise
    finally:
        print(f"# wall time {time.time() - t0:.1f} s", file=sys.stderr)


if __name__ == "__main__":
    main()
