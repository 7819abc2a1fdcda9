"""Architectures.  Importing this package registers them with `beglin_b200.config.registry`."""
from . import nadilorn, qwen2, sofudra, sukisun, tuzupel  # noqa: F401
