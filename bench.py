"""Headline benchmark: BERT-large masked-LM training throughput (samples/s).

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 10 --warmup 3

Config (the reference's BERT-large benchmark shape): 24 layers, hidden 1024,
16 heads, FFN 4096 GeLU, vocab 30522 (padded to a multiple of the TP size),
sequence 512, bf16, synthetic uniform token ids with 15 % masked labels,
random-init weights, 32 samples per GPU (global batch 256 on 8 GPUs),
activation checkpointing on every other layer, AdamW.  With N > 1 GPUs the
model is tensor-parallel over all N (TP = N, with sequence parallelism for
the native arm), i.e. weak scaling of the global batch.

Two arms:

* default: this framework (``apply_schedule`` -> ``build(target="native")``
  -> ``engine.train_batch``);
* ``--impl reference``: the unmodified reference package from
  ``baseline/_ref`` through its public API (``create_schedule`` / ``shard`` /
  ``sync`` / ``checkpoint`` / ``build``) on a Hugging Face ``BertForMaskedLM``
  with a plain PyTorch AdamW loop, which is what the reference's
  ``examples/utils.py`` does when no DeepSpeed / Megatron runtime exists.

Rank 0 prints ONE JSON line.  ``value`` is device-timed (CUDA events, max
over ranks) over exactly K steps with inputs resident on the device; ``e2e``
repeats the measurement through the public API including, every step, the
pinned-host -> device copy of the batch and a device -> host read of the loss.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(layers=24, hidden=1024, heads=16, ffn=4096, vocab=30522, seq=512)
# the second headline model: OPT-2.7B-shaped causal LM, sequence 1024, micro-batches of 4,
# 8 samples per GPU per step (global batch 64 on 8 GPUs, where the native arm runs the
# pipeline configuration PP 2 x TP 4 with 16 micro-batches)
OPT = dict(name="opt-2.7b", layers=32, hidden=2560, heads=32, ffn=10240, vocab=50272, seq=1024,
           micro_batch=4, batch_per_gpu=8)

# keys of the "config" object, identical for both arms (arm-specific remarks go to "notes")
CONFIG_KEYS = ("model", "layers", "global_batch", "seq_len", "parallelism", "ckpt_ratio",
               "optimizer", "micro_batch", "l2_policy")
L2_POLICY = ("per-step working set (weights+activations, >10 GB) exceeds the 126 MB L2, "
             "nothing survives between steps")


def make_config(model, layers, global_batch, seq_len, parallelism, ckpt_ratio, micro_batch):
    return {"model": model, "layers": layers, "global_batch": global_batch, "seq_len": seq_len,
            "parallelism": parallelism, "ckpt_ratio": ckpt_ratio, "optimizer": "AdamW",
            "micro_batch": micro_batch, "l2_policy": L2_POLICY}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default="bert-large", choices=["bert-large", "opt-2.7b"],
                    help="bert-large: the headline run; opt-2.7b: the second headline model "
                         "(same JSON line, metric 'train samples/sec, OPT-2.7B causal LM')")
    ap.add_argument("--with-opt", action="store_true",
                    help="after the BERT-large run also run OPT-2.7B and attach its record to "
                         "the JSON line under 'opt'")
    ap.add_argument("--batch-per-gpu", type=int, default=0, help="0 = the model's default")
    ap.add_argument("--seq", type=int, default=0, help="0 = the model's default")
    ap.add_argument("--layers", type=int, default=0, help="0 = the model's default")
    ap.add_argument("--ckpt-ratio", type=float, default=-1.0,
                    help="-1 = the model's default (bert-large 0.5, opt-2.7b 0)")
    ap.add_argument("--opt-layout", default="auto", choices=["auto", "tp", "pp2"],
                    help="opt-2.7b on 8 GPUs: pp2 = PP 2 x TP 4 (default), tp = TP 8")
    ap.add_argument("--no-tp-check", action="store_true",
                    help="skip the fused-vs-NCCL numerical check that multi-GPU runs do first")
    ap.add_argument("--parallelism", default="tp", choices=["tp", "dp"])
    ap.add_argument("--no-sequence-parallel", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cuda-graph", action="store_true",
                    help="single-GPU runs replay the whole step from one CUDA graph; this flag "
                         "launches the kernels one by one instead")
    ap.add_argument("--no-fused-dp", action="store_true",
                    help="data parallelism through NCCL instead of the peer-memory kernels")
    ap.add_argument("--watchdog", type=float, default=1500.0,
                    help="seconds after which a run that has not finished dumps every thread's "
                         "stack and exits with an error instead of blocking its caller (0 = off)")
    ap.add_argument("--profile", action="store_true",
                    help="print a per-kernel time table of one step (torch.profiler, rank 0); "
                         "analysis aid only, the reported numbers are taken without it")
    args = ap.parse_args()
    bert = args.model == "bert-large"
    args.batch_per_gpu = args.batch_per_gpu or (32 if bert else OPT["batch_per_gpu"])
    args.seq = args.seq or (MODEL["seq"] if bert else OPT["seq"])
    args.layers = args.layers or (MODEL["layers"] if bert else OPT["layers"])
    if args.ckpt_ratio < 0:
        args.ckpt_ratio = 0.5 if bert else 0.0
    return args


# --------------------------------------------------------------------------- #
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read only)."""

    def __init__(self, index, period=0.2):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(self.period)

    def finish(self):
        self._halt.set()
        if self.is_alive():
            self.join(timeout=2)
        med = sorted(self.samples)[len(self.samples) // 2] if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def make_batch(vocab, batch, seq, seed, device="cpu", pin=False):
    import torch

    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (batch, seq), generator=g)
    labels = torch.full_like(ids, -100)
    pick = torch.rand(batch, seq, generator=g) < 0.15
    labels[pick] = ids[pick]
    if pin:
        ids, labels = ids.pin_memory(), labels.pin_memory()
    return ids.to(device), labels.to(device)


def dist_setup(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def timed_loop(step_fn, steps, device, world):
    """Time exactly ``steps`` calls of ``step_fn`` on the device; max over ranks."""
    import torch
    import torch.distributed as dist

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(steps):
        step_fn(i)
    t1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = t0.elapsed_time(t1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


# --------------------------------------------------------------------------- #
def build_native(args, world, rank):
    import torch

    import slapo_b200 as slapo
    from slapo_b200.models import BertConfig, BertForMaskedLM, mlm_loss
    from slapo_b200.models.schedules.common import pad_vocab
    from slapo_b200.parallel.mesh import DeviceMesh

    tp = world if args.parallelism == "tp" else 1
    dp = world // tp
    mesh = DeviceMesh(pp=1, dp=dp, tp=tp) if world > 1 else None
    vocab = pad_vocab(MODEL["vocab"], 8 * tp if tp > 1 else 8)
    cfg = BertConfig(vocab_size=vocab, hidden_size=MODEL["hidden"],
                     num_hidden_layers=args.layers, num_attention_heads=MODEL["heads"],
                     intermediate_size=MODEL["ffn"], max_position_embeddings=max(512, args.seq))
    sp = tp > 1 and not args.no_sequence_parallel
    slapo.set_random_seed(2013, dp_rank=mesh.dp_rank if mesh else 0,
                          tp_rank=mesh.tp_rank if mesh else 0, always_enable_tp_seed=sp)
    with slapo.init_empty_weights():
        model = BertForMaskedLM(cfg)
    sch = slapo.model_schedule.apply_schedule(
        model, "bert", model_config=cfg, bf16=True, group=mesh.schedule_group if mesh else None,
        ckpt_ratio=args.ckpt_ratio, sequence_parallel=sp)
    vocab_parallel = tp > 1
    tp_group = mesh.tp_group if mesh else None

    def loss_fn(out, labels):
        return mlm_loss(out["logits"], labels, tp_group, vocab_parallel)

    engine, _ = slapo.build(sch, target="native", mesh=mesh, loss_fn=loss_fn,
                            config={"lr": 1e-4, "weight_decay": 0.01, "clip_grad": 1.0,
                                    "fused_dp": not args.no_fused_dp})
    parallelism = f"tp{tp}" + ("+sp" if sp else "") if tp > 1 else (f"dp{dp}" if dp > 1 else "single")
    return engine, vocab, parallelism, dp


def tp_numerical_check(world, device):
    """Before a tensor-parallel run is timed: the same 2-layer BERT-large-shaped model, same
    weights, same batch, once through the fused GEMM + collective kernels and once through
    this framework's NCCL ``sync`` ops; returns the relative differences of the loss and of the
    gradients (max over parameters of max|g_fused - g_nccl| / max|g_nccl|).  This is the
    evidence that the peer-memory path computes the right thing on real NVLink."""
    import torch

    import slapo_b200 as slapo
    from slapo_b200.models import BertConfig, BertForMaskedLM, mlm_loss
    from slapo_b200.models.schedules.common import pad_vocab
    from slapo_b200.parallel.mesh import DeviceMesh

    mesh = DeviceMesh(pp=1, dp=1, tp=world)
    vocab = pad_vocab(MODEL["vocab"], 8 * world)
    cfg = BertConfig(vocab_size=vocab, hidden_size=MODEL["hidden"], num_hidden_layers=2,
                     num_attention_heads=MODEL["heads"], intermediate_size=MODEL["ffn"],
                     max_position_embeddings=512, hidden_dropout_prob=0.0,
                     attention_probs_dropout_prob=0.0)
    ids, labels = make_batch(vocab, 4 * world, 512, 4321, device)
    runs = []
    for fused in (True, False):
        slapo.set_random_seed(77, dp_rank=0, tp_rank=mesh.tp_rank, always_enable_tp_seed=True)
        with slapo.init_empty_weights():
            model = BertForMaskedLM(cfg)
        sch = slapo.model_schedule.apply_schedule(
            model, "bert", model_config=cfg, bf16=True, group=mesh.schedule_group,
            ckpt_ratio=0.0, sequence_parallel=True)
        engine, _ = slapo.build(sch, target="native", mesh=mesh, fused_tp=fused,
                                config={"lr": 0.0, "clip_grad": 0.0})
        out = engine(ids)
        loss = mlm_loss(out["logits"], labels, mesh.tp_group, True)
        loss.backward()
        torch.cuda.synchronize()
        runs.append((float(loss), [p.grad.detach().float().clone() for p in engine.params]))
        del engine, model, sch, out, loss
    (l_f, g_f), (l_n, g_n) = runs
    grad_err = 0.0
    for a, b in zip(g_f, g_n):
        denom = float(b.abs().max())
        if denom > 0:
            grad_err = max(grad_err, float((a - b).abs().max()) / denom)
    t = torch.tensor([abs(l_f - l_n) / max(abs(l_n), 1e-6), grad_err], device=device)
    import torch.distributed as dist

    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    torch.cuda.empty_cache()
    return {"loss_fused": l_f, "loss_nccl": l_n, "loss_rel_err": float(t[0]),
            "grad_max_rel_err": float(t[1]), "ok": bool(t[0] < 2e-2 and t[1] < 2e-2),
            "model": "2-layer bert-large shape, 4 samples x 512 tokens per rank, tp+sp"}


def run_native(args):
    import torch

    from slapo_b200.ops import native

    if args.model == "opt-2.7b":
        return run_native_opt(args)
    world, rank, local = dist_setup(args)
    device = torch.device("cuda", local)
    tp_check = None
    if world > 1 and args.parallelism == "tp" and not args.no_tp_check \
            and not args.no_sequence_parallel:
        tp_check = tp_numerical_check(world, device)
        if rank == 0 and not tp_check["ok"]:
            print(f"# WARNING: fused and NCCL tensor-parallel paths disagree: {tp_check}",
                  file=sys.stderr)
        if max(tp_check["loss_rel_err"], tp_check["grad_max_rel_err"]) > 0.1:
            raise RuntimeError(f"fused tensor-parallel kernels give wrong results: {tp_check}")
    engine, vocab, parallelism, dp = build_native(args, world, rank)
    tp = world // dp
    # TP ranks consume the same batch; DP replicas different ones
    local_batch = args.batch_per_gpu * tp
    dp_rank = rank // tp
    ids, labels = make_batch(vocab, local_batch, args.seq, 1234 + dp_rank, device)
    global_batch = local_batch * dp

    graphed = None
    if world == 1 and not args.no_cuda_graph and not args.profile:
        try:
            graphed = engine.capture_step(ids, labels=labels, warmup=max(args.warmup, 3))
        except Exception as err:  # fall back to launching kernel by kernel
            print(f"# CUDA graph capture failed, running eagerly: {type(err).__name__}: {err}",
                  file=sys.stderr)
            graphed = None
            torch.cuda.synchronize()

    def step(_i):
        if graphed is not None:
            graphed(ids, labels=labels)
        else:
            engine.train_batch(ids, labels=labels)

    args.cuda_graph_used = graphed is not None
    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = native.launch_count()
    ms = timed_loop(step, args.steps, device, world)
    launches = native.launch_count() - launches0
    if graphed is not None:   # kernels inside the replayed graph are not counted by the host
        launches = graphed.kernels_per_step * args.steps
    clocks = sampler.finish()
    value = global_batch * args.steps / (ms / 1e3)

    if args.profile:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            step(0)
            torch.cuda.synchronize()
        if rank == 0:
            print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40,
                                            max_name_column_width=70), file=sys.stderr)
            # device kernels only: total ms, launches, name
            rows = [(e.device_time_total / 1e3, e.count, e.key) for e in prof.key_averages()
                    if getattr(e, "device_type", None) is not None
                    and "cuda" in str(e.device_type).lower() and e.device_time_total > 0]
            rows.sort(reverse=True)
            print("# device kernels of one step (ms, launches, name); sum = "
                  f"{sum(r[0] for r in rows):.2f} ms", file=sys.stderr)
            for ms_k, cnt, key in rows[:45]:
                print(f"#   {ms_k:9.3f} {cnt:5d}  {key[:110]}", file=sys.stderr)
    e2e = None
    losses = []
    if not args.no_e2e:
        host = [make_batch(vocab, local_batch, args.seq, 77 + dp_rank * 100 + i, "cpu", pin=True)
                for i in range(2)]
        h2d = sum(t.numel() * t.element_size() for t in host[0])

        def e2e_step(i):
            hi, hl = host[i % 2]
            di = hi.to(device, non_blocking=True)
            dl = hl.to(device, non_blocking=True)
            loss = graphed(di, labels=dl) if graphed is not None else \
                engine.train_batch(di, labels=dl)
            losses.append(float(loss.item()))  # device -> host read of the result
            return losses[-1]

        e2e_step(0)
        ms_e = timed_loop(e2e_step, args.steps, device, world)
        e2e = {"value": global_batch * args.steps / (ms_e / 1e3), "unit": "samples/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
               "ms_per_step": ms_e / args.steps}
    getattr(engine, "check_device_status", lambda: None)()
    opt_record = None
    if args.with_opt:
        del engine, graphed
        torch.cuda.empty_cache()
        opt_record = run_native_opt(args, setup=(world, rank, local), emit=False)
    if rank == 0:
        print(json.dumps({
            "metric": "train samples/sec, BERT-large MLM", "value": value, "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "native",
            "config": make_config("bert-large", args.layers, global_batch, args.seq,
                                  parallelism.replace("+sp", ""), args.ckpt_ratio, local_batch),
            "notes": {"sequence_parallel": "+sp" in parallelism,
                      "attention": "tcgen05 flash attention (this library)",
                      "gemm": "tcgen05 GEMM (this library); fused GEMM + collective under TP"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
            "cuda_graph": args.cuda_graph_used,
            "loss": {"first": losses[0] if losses else None, "last": losses[-1] if losses else None,
                     "steps_trained_before_last": args.warmup * 2 + args.steps * 2},
            "tp_check": tp_check, "opt": opt_record,
            "max_mem_mb": torch.cuda.max_memory_allocated() / 2**20,
        }), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


# --------------------------------------------------------------------------- #
def opt_layout(world, choice):
    """(tp, pp) of the OPT-2.7B run on ``world`` GPUs: tensor parallel over all of them, except
    on 8 GPUs where the target configuration is 2 pipeline stages of 4-way tensor parallelism."""
    if world == 8 and choice in ("auto", "pp2"):
        return 4, 2
    return world, 1


def run_native_opt(args, setup=None, emit=True):
    """OPT-2.7B-shaped causal LM through the same public API (zoo spec -> ``apply_schedule`` ->
    ``build(target="native")`` -> ``engine.train_batch``), micro-batches of 4 x 1024 tokens."""
    import argparse as _argparse

    import torch

    from slapo_b200.bench.train import build_engine
    from slapo_b200.ops import native

    world, rank, local = setup if setup is not None else dist_setup(args)
    device = torch.device("cuda", local)
    tp, pp = opt_layout(world, args.opt_layout)
    micro = OPT["micro_batch"]
    per_gpu = OPT["batch_per_gpu"] if args.model != "opt-2.7b" else args.batch_per_gpu
    global_batch = per_gpu * world
    n_micro = max(global_batch // micro, 1)
    layers = OPT["layers"] if args.model != "opt-2.7b" else args.layers
    seq = OPT["seq"] if args.model != "opt-2.7b" else args.seq
    ckpt = 0.0 if args.model != "opt-2.7b" else args.ckpt_ratio
    targs = _argparse.Namespace(
        model="opt-2.7b", tp=tp, pp=pp, dp=1, batch_size=micro, micro_batches=n_micro,
        seq_len=seq, seq_len_dec=0, layers=layers if layers != OPT["layers"] else 0, hidden=0,
        heads=0, vocab=0, ckpt_ratio=ckpt, sequence_parallel=tp > 1, no_fuse=False,
        attn_op="auto", dtype="bf16", lr=1e-4, seed=2013, no_fused_dp=False)
    engine, spec, mesh, dp = build_engine(targs, world, device)
    per_call = micro * (n_micro if pp > 1 else 1)
    calls = 1 if pp > 1 else n_micro
    batches = [spec.make_batch(per_call, seq, 0, seed=2013 + i, device=device) for i in range(calls)]

    def step(_i):
        loss = None
        for inputs, labels in batches:
            loss = engine.train_batch(*inputs, labels=labels)
        return loss

    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = native.launch_count()
    ms = timed_loop(step, args.steps, device, world)
    launches = native.launch_count() - launches0
    clocks = sampler.finish()
    value = global_batch * args.steps / (ms / 1e3)
    e2e, losses = None, []
    if not args.no_e2e:
        host = [[spec.make_batch(per_call, seq, 0, seed=4000 + 10 * j + i, device="cpu", pin=True)
                 for i in range(calls)] for j in range(2)]
        h2d = sum(t.numel() * t.element_size() for inputs, labels in host[0]
                  for t in list(inputs) + [labels])

        def e2e_step(i):
            loss = None
            for inputs, labels in host[i % 2]:
                dev_in = [t.to(device, non_blocking=True) for t in inputs]
                loss = engine.train_batch(*dev_in, labels=labels.to(device, non_blocking=True))
            losses.append(float(loss.item()))
            return losses[-1]

        e2e_step(0)
        ms_e = timed_loop(e2e_step, args.steps, device, world)
        e2e = {"value": global_batch * args.steps / (ms_e / 1e3), "unit": "samples/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * calls,
               "ms_per_step": ms_e / args.steps}
    getattr(getattr(engine, "inner", engine), "check_device_status", lambda: None)()
    # model FLOPs per sample (the reference's formula: 3 x (L (4 h s^2 + 24 s h^2) + 2 s h v))
    h_, s_, v_ = OPT["hidden"], seq, OPT["vocab"]
    flops = 3.0 * (layers * (4 * h_ * s_ * s_ + 24 * s_ * h_ * h_) + 2 * s_ * h_ * v_)
    parallelism = (f"pp{pp}xtp{tp}" if pp > 1 else (f"tp{tp}" if tp > 1 else "single"))
    record = {
        "metric": "train samples/sec, OPT-2.7B causal LM", "value": value, "unit": "samples/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "native",
        "config": make_config("opt-2.7b", layers, global_batch, seq, parallelism, ckpt, micro),
        "notes": {"sequence_parallel": tp > 1, "micro_batches": n_micro,
                  "attention": "tcgen05 flash attention, head dim 80 (this library)"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "cuda_graph": False,
        "loss": {"first": losses[0] if losses else None, "last": losses[-1] if losses else None},
        "model_tflops_per_gpu": flops * value / world / 1e12,
        "max_mem_mb": torch.cuda.max_memory_allocated() / 2**20,
    }
    if emit:
        if rank == 0:
            print(json.dumps(record), flush=True)
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()
    return record


# --------------------------------------------------------------------------- #
def run_reference(args):
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "slapo")):
        print(json.dumps({"impl": "reference",
                          "unavailable": "baseline/_ref is missing (offline pip install not done)"}))
        return
    try:
        from baseline.reference_arm import run
    except Exception as err:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"harness import failed: {err}"}))
        return
    if args.model == "opt-2.7b":
        from baseline.reference_arm import run_opt

        run_opt(args, ref_root, OPT, dist_setup, timed_loop, ClockSampler, make_config)
        return
    run(args, ref_root, MODEL, dist_setup, make_batch, timed_loop, ClockSampler, make_config)


def maybe_self_launch(args):
    """``python bench.py --gpus N`` without torchrun: start the ranks ourselves."""
    if args.gpus > 1 and "RANK" not in os.environ:
        port = 29500 + (os.getpid() % 2000)
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
               "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))


def main():
    args = parse_args()
    maybe_self_launch(args)
    if args.watchdog > 0:
        import faulthandler

        # a rank that hangs (a peer that never arrives, a lost transfer) must not hang the caller
        faulthandler.dump_traceback_later(args.watchdog, exit=True, file=sys.stderr)
    try:
        if args.impl == "reference":
            run_reference(args)
        else:
            run_native(args)
    finally:
        if args.watchdog > 0:
            import faulthandler

            faulthandler.cancel_dump_traceback_later()


if __name__ == "__main__":
    main()
