"""Auto-tune every model of a list on N GPUs of this machine, one after the other.

    python benchmark/tune_single_node.py --gpus 8 --models bert-large opt-350m t5-large

For each model it runs ``python -m slapo_b200.autotune.tune`` with the family's
``examples/<family>/tune_cfg.py`` around ``benchmark/bench_single_node.py run``
and stores every evaluated point in ``<model>-gpu<N>.json``.  With ``--gpus 1``
it is the single-device driver.  (benchmark/tune_single_node.py:6-46 and
tune_single_device.py:6-44 of the reference do the same over Megatron /
DeepSpeed launch lines.)
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def family_of(model):
    from slapo_b200.models.zoo import get_model_spec

    return get_model_spec(model).schedule_key


def tune_command(model, gpus, tp, seq, db, extra=()):
    cfg = os.path.join(ROOT, "examples", family_of(model), "tune_cfg.py")
    return [sys.executable, "-m", "slapo_b200.autotune.tune", "--config", cfg, "--db", db,
            "--error-stop", "symbol", os.path.join(ROOT, "benchmark", "bench_single_node.py"),
            "run", "--model", model, "--gpus", str(gpus), "--tp", str(tp), "--seq-len", str(seq),
            "--batch-size", "batch_size", "--ckpt-ratio", "ckpt_ratio", *extra]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--tp", type=int, default=0, help="0 = all GPUs")
    ap.add_argument("--models", nargs="+", default=["bert-large", "roberta-large", "albert-large",
                                                    "opt-350m", "gpt-neo-1.3b", "t5-large"])
    ap.add_argument("--out-dir", default=".")
    ap.add_argument("--dry-run", action="store_true", help="print the commands only")
    ns = ap.parse_args(argv)
    from slapo_b200.models.zoo import get_model_spec

    for model in ns.models:
        spec = get_model_spec(model)
        db = os.path.join(ns.out_dir, f"{model}-gpu{ns.gpus}.json")
        cmd = tune_command(model, ns.gpus, ns.tp or ns.gpus, spec.default_seq, db)
        print(" ".join(cmd), flush=True)
        if not ns.dry_run:
            subprocess.run(cmd, cwd=ROOT, check=False,
                           env=dict(os.environ, PYTHONPATH=ROOT))


if __name__ == "__main__":
    main()
