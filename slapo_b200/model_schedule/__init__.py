"""Per-model scheduling recipes; importing the package registers all of them."""
from .api import apply_schedule  # noqa: F401
from .registry import SCHEDULE_METHODS, get_schedule, register_schedule  # noqa: F401
from ..models import schedules as _schedules  # noqa: F401,E402  (registers the recipes)
