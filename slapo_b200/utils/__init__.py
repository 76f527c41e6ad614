"""Utilities: hook plumbing, functional/module maps, reports, versions."""
from . import common, mapping, report, versions  # noqa: F401
