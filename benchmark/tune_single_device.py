"""Auto-tune the single-device benchmark models, one after the other, on ONE GPU.

    python benchmark/tune_single_device.py [--models bert-large opt-350m ...] [--dry-run]

The single-device counterpart of ``tune_single_node.py``: the same tuner
(``python -m slapo_b200.autotune.tune`` with the family's ``examples/<family>/tune_cfg.py``)
around ``benchmark/bench_single_node.py run --gpus 1``, searching batch size and checkpoint
ratio, one JSON database per model (``<model>-gpu1.json``).  The model list is the reference's
single-device list (benchmark/tune_single_device.py:6-44 of the reference: BERT-large,
RoBERTa-large, GPT-Neo-125M, OPT-350M, T5-base, WideResNet-250M), sequence length 1024 for the
decoder-style models and 512 otherwise.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import tune_single_node  # noqa: E402

MODELS = ["bert-large", "roberta-large", "gpt-neo-125m", "opt-350m", "t5-base", "wideresnet-250M"]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--models", nargs="+", default=MODELS)
    ap.add_argument("--out-dir", default=".")
    ap.add_argument("--dry-run", action="store_true", help="print the commands only")
    ns = ap.parse_args(argv)
    args = ["--gpus", "1", "--tp", "1", "--models", *ns.models, "--out-dir", ns.out_dir]
    if ns.dry_run:
        args.append("--dry-run")
    tune_single_node.main(args)


if __name__ == "__main__":
    main()
