"""Architectures known to the registry."""
from . import qwen2, rolesun  # noqa: F401
