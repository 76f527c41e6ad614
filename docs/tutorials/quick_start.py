"""Quick start: schedule a model without touching its source
===========================================================

Runs on CPU in a few seconds::

    python docs/tutorials/quick_start.py

A *schedule* is a tree that mirrors the module hierarchy of a model.  Every node offers the
scheduling primitives as methods; a primitive rewrites the module in place (replace it, shard
its parameters, checkpoint it, ...) and never edits the model's Python source.  ``build`` turns
the schedule back into an ordinary ``nn.Module`` - or, with ``target="native"``, into this
framework's training engine.
"""
import os
import sys

import torch
from torch import nn

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import slapo_b200 as slapo  # noqa: E402


# %% A model written with no thought for performance or parallelism.
class Block(nn.Module):
    def __init__(self, width):
        super().__init__()
        self.fc1 = nn.Linear(width, 4 * width)
        self.act = nn.GELU()
        self.fc2 = nn.Linear(4 * width, width)
        self.norm = nn.LayerNorm(width)

    def forward(self, x):
        return self.norm(x + self.fc2(self.act(self.fc1(x))))


class Net(nn.Module):
    def __init__(self, width=32, depth=3):
        super().__init__()
        self.blocks = nn.ModuleList([Block(width) for _ in range(depth)])
        self.head = nn.Linear(width, 8)

    def forward(self, x):
        for blk in self.blocks:
            x = blk(x)
        return self.head(x)


def main():
    torch.manual_seed(0)
    model = Net()
    x = torch.randn(4, 10, 32)
    want = model(x)

    # %% Create the schedule and look around.  Elements of a ModuleList are one path token.
    sch = slapo.create_schedule(model)
    print("primitives:", slapo.list_primitives())
    print("children of the root:", list(sch.child))
    print("a node:", sch["blocks.0.fc1"])

    # %% Primitive 1 - replace: swap a module for another one with the same call signature.
    #    Here: the two-kernel "Linear then GELU" becomes one module whose bias add and
    #    activation run fused (on CUDA: in this library's kernels; on CPU: plain PyTorch).
    from slapo_b200.ops.linear import LinearWithAct

    for i in range(3):
        blk = sch[f"blocks.{i}"]
        fused = LinearWithAct.from_linear(blk["fc1"].mod, act_fn="gelu")
        blk["fc1"].replace(fused)
        blk["act"].replace(nn.Identity())

    # %% Primitive 2 - checkpoint: recompute a block's activations in backward.
    sch["blocks.1"].checkpoint()

    # %% Primitive 3 - annotate: attach a tag to a parameter; it survives build() and the
    #    training engine reads tags such as "replicated_param".
    sch["head"].annotate("bias", "no_weight_decay", True)

    # %% build() hands back the scheduled model.  Nothing was copied: the parameters are the
    #    very objects of the original model.
    built, _ = slapo.build(sch, init_weights=False)
    print(built.blocks[1])
    torch.testing.assert_close(built(x), want, rtol=1e-5, atol=1e-5)
    assert built.head.weight is model.head.weight and built.head.bias.no_weight_decay

    # %% The same schedule drives the native training engine.
    engine, _ = slapo.build(slapo.create_schedule(built), target="native", init_weights=False,
                            config={"lr": 1e-2},
                            loss_fn=lambda out, labels: (out - labels).pow(2).mean())
    y = torch.randn(4, 10, 8)
    losses = [float(engine.train_batch(x, labels=y)) for _ in range(5)]
    print("training losses:", [round(v, 4) for v in losses])
    assert losses[-1] < losses[0]
    print("quick start finished")


if __name__ == "__main__":
    main()
