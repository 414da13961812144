"""Architectures: each module turns its configuration into a plan and registers itself."""
from . import llama, rigitar  # noqa: F401
