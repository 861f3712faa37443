"""Architectures known to the registry."""
from . import qwen2, retodra, rolesun  # noqa: F401
