"""Architectures.  Importing this package registers them."""

from . import llama, namalix, revirax, tefavik, vezatar  # noqa: F401
