"""Per-model scheduling recipes (registered on import)."""
from . import bert  # noqa: F401
