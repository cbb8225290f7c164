"""Architectures.  Importing this package registers every architecture it holds."""

from . import gulazen, kudazen, nazulorn, paditar, qwen3  # noqa: F401
