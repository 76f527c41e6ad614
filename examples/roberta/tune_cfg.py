"""Auto-tuning configuration for roberta-large: the batch-size range searched per
GPU count; the tuner then searches the checkpoint ratio for each batch size.

    python -m slapo_b200.autotune.tune --config examples/roberta/tune_cfg.py --db roberta-gpu8.json \
        benchmark/bench_single_node.py run --model roberta-large --gpus 8 --tp 8 \
            --seq-len 512 --batch-size batch_size --ckpt-ratio ckpt_ratio

``batch_size`` and ``ckpt_ratio`` in the command are symbols that the tuner
substitutes for each trial.  Ranges assume 180 GB of HBM3e per GPU.
"""


def get_bs_range(args):
    n_gpu = int(args.get("gpus", 1))
    tp = int(args.get("tp", 1))
    dp = max(1, n_gpu // tp)
    base = 32
    min_bs = base // 2 if base >= 2 else 1
    max_bs = base * 8
    step = max(1, min_bs)
    return (min_bs, max_bs, step)


def is_valid(args, cfg):
    """Skip points that cannot run: the micro-batch must split evenly."""
    micro = int(args.get("micro-batches", 1))
    return cfg["batch_size"] >= 1 and cfg["batch_size"] % 1 == 0 and micro >= 1
