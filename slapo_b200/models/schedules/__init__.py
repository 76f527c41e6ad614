"""Per-model scheduling recipes (registered on import)."""
from . import albert, bert, decoder, t5, wideresnet  # noqa: F401
