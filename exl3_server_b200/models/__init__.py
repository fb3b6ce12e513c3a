"""Architectures: each module turns its configuration into a plan and registers itself."""
from . import llama, nibelix, nikodra, potodra, rigitar  # noqa: F401
