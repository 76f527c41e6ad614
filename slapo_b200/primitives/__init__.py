"""Schedule primitives.  Importing this package registers the built-in ones;
third-party primitives register themselves with ``@register_primitive()``."""
from .base import PRIMITIVES, Primitive, register_primitive  # noqa: F401
from . import annotate, checkpoint, fusion, pipeline, replace, tensor_parallel  # noqa: F401,E402
