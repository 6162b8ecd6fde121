"""Architectures this library ships.  Importing the package registers them."""

from . import qwen2  # noqa: F401  (registration)
