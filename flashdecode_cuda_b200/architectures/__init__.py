"""Architectures this library ships.  Importing the package registers them."""

from . import botusun, lonasun, nizazen, qwen2, revelix  # noqa: F401  (registration)
