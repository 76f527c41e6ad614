"""Alias of :mod:`slapo_b200.ops` under the reference's module name ``op``."""
from .ops import *  # noqa: F401,F403
from .ops import attention, cross_entropy, functional, linear, mlp, norm, utils  # noqa: F401
