"""Train gpt2-medium (or another size of the family via ``--model``) on synthetic data
with the native engine.

    python examples/gpt2/train.py --steps 20                              # one GPU
    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        examples/gpt2/train.py --tp 8 --sequence-parallel --batch-size 8 --ckpt-ratio 0.5

Every flag of ``slapo_b200.bench.train`` applies (``--tp --pp --dp --batch-size
--micro-batches --seq-len --ckpt-ratio --save --resume ...``).
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from slapo_b200.bench.train import main  # noqa: E402

if __name__ == "__main__":
    argv = sys.argv[1:]
    if "--model" not in argv:
        argv = ["--model", "gpt2-medium"] + argv
    if "--seq-len" not in argv:
        argv += ["--seq-len", "1024"]
    main(argv)
