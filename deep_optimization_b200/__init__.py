"""B200-native activation-compression kernels behind Deep_Optimization's operator API."""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
