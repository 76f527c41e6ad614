"""Runtime adapters; importing the package registers the built-in ones."""
from .registry import (DIALECTS, get_all_dialects, get_dialect_cls,  # noqa: F401
                       register_framework_dialect)
from . import log_parsers  # noqa: F401,E402
from . import native  # noqa: F401,E402
from . import compat  # noqa: F401,E402
