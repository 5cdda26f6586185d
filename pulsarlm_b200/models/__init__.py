"""Architectures: importing this package registers every one of them."""

from . import llama, rerilorn  # noqa: F401
