"""slapo_b200: a B200-native schedule language for large-model training.

The public surface follows awslabs/slapo (``create_schedule`` -> primitives ->
``build``); underneath, the hot paths are hand-written sm_100a kernels and the
runtime (data/tensor/sequence/pipeline parallel engines, checkpoint I/O,
solver, auto-tuner) is part of the package.
"""
from .version import __version__  # noqa: F401
from . import primitives  # noqa: F401  (registers the built-in primitives)
from .primitives.base import Primitive, register_primitive  # noqa: F401
from .schedule import Schedule, create_schedule, list_primitives  # noqa: F401
from .build import build  # noqa: F401
from .verify import Verify  # noqa: F401
from .checkpoint import checkpoint  # noqa: F401
from .random import get_cuda_rng_tracker, is_random_seed_set, set_random_seed  # noqa: F401
from .initialization import init_empty_weights  # noqa: F401
from .logger import get_logger  # noqa: F401
from .autotune.tune import Database, Space, Symbol  # noqa: F401
from . import env, op, pattern, pipeline, sharding, tracer  # noqa: F401,E402
from . import framework_dialect, model_schedule, models  # noqa: F401,E402
from .parallel.mesh import DeviceMesh  # noqa: F401
