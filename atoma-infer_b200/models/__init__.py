"""Architectures built from the parts; importing this package registers them."""
from . import llama  # noqa: F401
