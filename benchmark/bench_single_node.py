"""Single-node benchmark sweep over the model zoo.

    python benchmark/bench_single_node.py run --model bert-large --gpus 8 --tp 8 \
        --seq-len 512 --batch-size 32 --ckpt-ratio 0.5
    python benchmark/bench_single_node.py sweep --config benchmark/configs/single_node_b200.cfg \
        --out results.tsv

``run`` launches ``slapo_b200.bench.train`` on ``--gpus`` ranks of this machine
(torchrun, rendezvous on 127.0.0.1) and prints its JSON record; ``sweep`` does
so for every line of a config file.  A config line reads

    MODEL  GPUS  SEQ  SEQ_DEC  BATCH_EXPR  CKPT  [key=value ...]

with ``GPUS`` a comma list (``1,2,4,8``), ``BATCH_EXPR`` a Python expression of
``n`` (the GPU count) giving the global batch size, and optional ``tp=``, ``pp=``,
``micro=``, ``sp=1`` settings (``tp=n`` means "all GPUs").  One row per run is
appended to the TSV: model, GPUs, layout, batch, samples/s, model TFLOP/s per
GPU, peak memory.  It mirrors benchmark/bench_single_node.py:222-330 of the
reference, with the native engine in place of Megatron / DeepSpeed.
"""
from __future__ import annotations

import argparse
import json
import os
import shlex
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def model_tflop_per_sample(name, seq, seq_dec=0):
    """Model (not hardware) TFLOPs to train one sample: 3 x forward, attention
    included, checkpoint recompute excluded."""
    from slapo_b200.models.zoo import get_model_spec

    spec = get_model_spec(name)
    cfg = spec.config
    if spec.kind == "image":
        return 0.0
    get = lambda *keys: max(getattr(cfg, k, 0) or 0 for k in keys)  # noqa: E731
    n, h, v = spec.num_layers, get("hidden_size", "d_model"), cfg.vocab_size
    if spec.kind != "seq2seq":
        ffn = get("intermediate_size", "ffn_dim") or 4 * h
        att = 4 * h * seq**2 + 8 * seq * h**2
        forward = n * (att + 4 * seq * h * ffn) + 2 * seq * h * v
        return 3 * forward / 1e12
    inner, ff = cfg.num_heads * cfg.d_kv, cfg.d_ff
    gate = 3 if cfg.is_gated_act else 2
    enc = n * (8 * seq * h * inner + 4 * inner * seq**2 + 2 * gate * seq * h * ff)
    dec = cfg.num_decoder_layers * (
        8 * seq_dec * h * inner + 4 * inner * seq_dec**2               # self attention
        + 4 * seq_dec * h * inner + 4 * seq * h * inner + 4 * inner * seq * seq_dec  # cross
        + 2 * gate * seq_dec * h * ff) + 2 * seq_dec * h * v
    return 3 * (enc + dec) / 1e12


def launch(model, gpus, train_args, port=29540, timeout=None, env=None):
    """Run the training entry on ``gpus`` ranks; returns (record or None, log text)."""
    cmd = [sys.executable]
    if gpus > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}",
                "--master-addr", "127.0.0.1", "--master-port", str(port)]
    cmd += ["-m", "slapo_b200.bench.train", "--model", model] + list(train_args)
    full_env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    full_env.update(env or {})
    try:
        proc = subprocess.run(cmd, cwd=ROOT, env=full_env, text=True, capture_output=True,
                              timeout=timeout, check=False)
        text = proc.stdout + proc.stderr
    except subprocess.TimeoutExpired as err:
        text = (err.stdout or "") + (err.stderr or "") + "\nTIMEOUT\n"
    record = None
    for line in text.splitlines():
        line = line.strip()
        if line.startswith("{") and '"samples_per_sec"' in line:
            try:
                record = json.loads(line)
            except json.JSONDecodeError:
                pass
    return record, text


def parse_config(path):
    runs = []
    with open(path, encoding="utf-8") as fh:
        for raw in fh:
            line = raw.split("#", 1)[0].strip()
            if not line:
                continue
            parts = shlex.split(line)
            model, gpus, seq, seq_dec, batch_expr, ckpt = parts[:6]
            opts = dict(p.split("=", 1) for p in parts[6:])
            for n in (int(g) for g in gpus.split(",")):
                batch = int(eval(batch_expr, {"min": min, "max": max}, {"n": n}))  # noqa: S307
                resolve = lambda v: n if v == "n" else int(v)  # noqa: E731
                tp = resolve(opts.get("tp", "n"))
                pp = resolve(opts.get("pp", "1"))
                tp = min(tp, max(1, n // pp))
                runs.append(dict(model=model, gpus=n, seq=int(seq), seq_dec=int(seq_dec),
                                 batch=batch, ckpt=float(ckpt), tp=tp, pp=pp,
                                 micro=int(opts.get("micro", "1")), sp=opts.get("sp", "0") == "1"))
    return runs


def train_args_for(run, steps, warmup):
    dp = run["gpus"] // (run["tp"] * run["pp"])
    per_replica = max(1, run["batch"] // max(dp, 1) // run["micro"])
    args = ["--tp", str(run["tp"]), "--pp", str(run["pp"]), "--batch-size", str(per_replica),
            "--micro-batches", str(run["micro"]), "--seq-len", str(run["seq"]),
            "--ckpt-ratio", str(run["ckpt"]), "--steps", str(steps), "--warmup", str(warmup)]
    if run["seq_dec"]:
        args += ["--seq-len-dec", str(run["seq_dec"])]
    if run["sp"]:
        args.append("--sequence-parallel")
    return args


def cmd_run(ns, extra):
    record, text = launch(ns.model, ns.gpus, extra, port=ns.port, timeout=ns.timeout)
    if record is None:
        sys.stdout.write(text[-4000:])
        sys.exit(1)
    record["model_tflops_per_gpu"] = (
        model_tflop_per_sample(ns.model, record["seq_len"], 0) * record["samples_per_sec"] / ns.gpus)
    print(json.dumps(record))


def cmd_sweep(ns, _extra):
    header = "model\tgpus\tlayout\tglobal_batch\tckpt\tsamples_per_sec\tmodel_tflops_per_gpu\tmax_mem_mb"
    rows = [header]
    for i, run in enumerate(parse_config(ns.config)):
        if ns.only and ns.only not in run["model"]:
            continue
        record, text = launch(run["model"], run["gpus"], train_args_for(run, ns.steps, ns.warmup),
                              port=ns.port + i % 50, timeout=ns.timeout)
        layout = f"tp{run['tp']}pp{run['pp']}dp{run['gpus'] // (run['tp'] * run['pp'])}"
        if record is None:
            oom = "OutOfMemoryError" in text
            rows.append(f"{run['model']}\t{run['gpus']}\t{layout}\t{run['batch']}\t{run['ckpt']}\t"
                        f"{'oom' if oom else 'fail'}\t0\t0")
        else:
            tfl = model_tflop_per_sample(run["model"], run["seq"], run["seq_dec"]) \
                * record["samples_per_sec"] / run["gpus"]
            rows.append(f"{run['model']}\t{run['gpus']}\t{layout}\t{run['batch']}\t{run['ckpt']}\t"
                        f"{record['samples_per_sec']:.2f}\t{tfl:.1f}\t{record['max_mem_mb']:.0f}")
        print(rows[-1], flush=True)
    if ns.out:
        with open(ns.out, "w", encoding="utf-8") as fh:
            fh.write("\n".join(rows) + "\n")


def cmd_env(ns, _extra):
    """Versions and devices of this machine, one ``key<TAB>value`` line each (the header block of
    a results file).  Parity: the ``env`` sub-command of the reference's bench_single_node.py."""
    import platform

    import torch

    rows = [("python", platform.python_version()), ("torch", torch.__version__),
            ("cuda (torch)", str(torch.version.cuda)), ("platform", platform.platform())]
    try:
        import slapo_b200
        from slapo_b200.ops import native

        rows.append(("slapo_b200", getattr(slapo_b200, "__version__", "in-tree")))
        rows.append(("native extension",
                     "loaded" if native.available() else f"missing: {native.load_error()}"))
    except Exception as err:        # the report must not fail on a broken install
        rows.append(("slapo_b200", f"import failed: {err}"))
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            prop = torch.cuda.get_device_properties(i)
            rows.append((f"gpu{i}", f"{prop.name}, {prop.total_memory // 2**20} MiB, "
                                    f"{prop.multi_processor_count} SMs, sm_{prop.major}{prop.minor}"))
        try:
            rows.append(("nccl", ".".join(str(v) for v in torch.cuda.nccl.version())))
        except Exception:
            pass
    else:
        rows.append(("gpu", "none visible"))
    text = "\n".join(f"{k}\t{v}" for k, v in rows) + "\n"
    sys.stdout.write(text)
    if ns.append_to:
        with open(ns.append_to, "a", encoding="utf-8") as fh:
            fh.write(text)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    run = sub.add_parser("run", help="one run; unknown flags go to slapo_b200.bench.train")
    run.add_argument("--model", required=True)
    run.add_argument("--gpus", type=int, default=1)
    sweep = sub.add_parser("sweep")
    sweep.add_argument("--config", required=True)
    sweep.add_argument("--out", default=None)
    sweep.add_argument("--only", default=None, help="substring filter on the model name")
    sweep.add_argument("--steps", type=int, default=10)
    sweep.add_argument("--warmup", type=int, default=3)
    env = sub.add_parser("env", help="versions and devices of this machine")
    env.add_argument("--append-to", default=None, help="also append the report to this file")
    for p in (run, sweep):
        p.add_argument("--port", type=int, default=29540)
        p.add_argument("--timeout", type=float, default=1800)
    ns, extra = ap.parse_known_args(argv)
    {"run": cmd_run, "sweep": cmd_sweep, "env": cmd_env}[ns.cmd](ns, extra)


if __name__ == "__main__":
    main()
