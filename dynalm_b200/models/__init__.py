"""Architectures; importing this package registers them."""
from . import llama, todupel  # noqa: F401
