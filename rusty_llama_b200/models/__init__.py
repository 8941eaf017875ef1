"""Architectures.  Importing this package registers them."""

from . import llama, revirax, tefavik, vezatar  # noqa: F401
