"""Looking inside a scheduled model
==================================

    python docs/tutorials/debug_print.py

Three tools: the graph of a traced node, ``Print`` - a leaf module that survives tracing and
prints *run-time* values from inside a graph - and ``Verify`` around a group of primitives.
"""
import io
import os
import sys
from contextlib import redirect_stdout

import torch
import torch.nn.functional as F
from torch import nn

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import slapo_b200 as slapo  # noqa: E402
from slapo_b200 import op  # noqa: E402


class Model(nn.Module):
    def __init__(self):
        super().__init__()
        self.proj = nn.Linear(8, 8)
        self.print = op.Print()          # costs nothing unless called

    def forward(self, x):
        y = F.relu(self.proj(x))
        # inside a traced graph `y` is a proxy: an f-string would print "Proxy(relu)".  Values
        # passed as ARGUMENTS are formatted when the graph runs.
        y = self.print(y, "after relu: shape", y.shape, "mean", y.mean())
        return y * 2


def main():
    torch.manual_seed(0)
    model = Model()
    x = torch.randn(2, 8)
    sch = slapo.create_schedule(model)

    # 1. the graph of a node: what `find` patterns are matched against
    sch.trace()
    print(sch.mod.graph)
    sch.mod.graph.print_tabular() if hasattr(sch.mod.graph, "print_tabular") else None

    # 2. Print is a leaf: it is a call_module node of the graph and prints at run time
    assert "print" in [n.target for n in sch.mod.graph.nodes if n.op == "call_module"]
    buf = io.StringIO()
    with redirect_stdout(buf):
        out = sch.mod(x)
    print("captured:", buf.getvalue().strip())
    assert "after relu: shape torch.Size([2, 8])" in buf.getvalue()
    torch.testing.assert_close(out, F.relu(model.proj(x)) * 2)

    # 3. Verify: a wrong rewrite is reported where it is made
    class Wrong(nn.Module):
        def forward(self, t):
            return t + 1.0

    sch2 = slapo.create_schedule(Model())
    try:
        with slapo.Verify(sch2, [x], device="cpu"):
            sch2["proj"].replace(Wrong())
    except Exception as err:
        print("Verify:", str(err).splitlines()[0][:100])
    else:
        raise AssertionError("Verify should have failed")

    # 4. a replaced module says what it does
    from slapo_b200.ops.linear import LinearWithSyncFunc

    sch3 = slapo.create_schedule(Model())
    sch3["proj"].replace(LinearWithSyncFunc.from_linear(sch3["proj"].mod))
    print(sch3.mod)
    print("debugging tutorial finished")


if __name__ == "__main__":
    main()
