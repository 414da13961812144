"""Architectures: each module turns its configuration into a plan and registers itself."""
from . import llama, nikodra, rigitar  # noqa: F401
