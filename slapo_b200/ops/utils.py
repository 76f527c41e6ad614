"""Debug printing inside traced graphs.

``Print`` is a leaf module (never traced into): put ``x = self.print(x, "x:",
x)`` in a forward and the values are printed at run time even after the
module has been traced, because the call survives as a ``call_module`` node.
It returns its first argument, so the node stays alive only if that result
is used.

Parity: slapo/op/utils.py:10-51 of the reference.
"""
from torch import nn


class Print(nn.Module):
    traceable = False

    def forward(self, tensor, *values, **kwargs):
        """Print ``values`` (evaluated lazily at run time) and return ``tensor``."""
        print(*values, **kwargs)
        return tensor
