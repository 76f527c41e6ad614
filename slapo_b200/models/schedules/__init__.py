"""Per-model scheduling recipes (registered on import)."""
from . import bert, decoder  # noqa: F401
