"""Placeholder so `import auto_precision` resolves: the reference's file of this name is
empty (Activation_Compression/auto_precision.py, 0 bytes).  The only auto-precision
arithmetic of the reference is the greedy allocator, exposed as `calc_precision`."""
from .codec import calc_precision  # noqa: F401
