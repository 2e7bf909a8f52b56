"""Architectures this library knows; importing the package registers them."""
from . import fusazen, garodra, llama  # noqa: F401
