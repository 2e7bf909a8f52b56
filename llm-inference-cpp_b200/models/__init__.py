"""Architectures this library knows; importing the package registers them."""
from . import garodra, llama  # noqa: F401
