"""Architectures; importing this package registers them."""
from . import llama, rematar, todupel  # noqa: F401
