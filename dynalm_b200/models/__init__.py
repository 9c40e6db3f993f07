"""Architectures; importing this package registers them."""
from . import bugapel, llama, rematar, rodelorn, todupel  # noqa: F401
