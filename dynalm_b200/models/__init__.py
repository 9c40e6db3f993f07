"""Architectures; importing this package registers them."""
from . import llama, rematar, rodelorn, todupel  # noqa: F401
