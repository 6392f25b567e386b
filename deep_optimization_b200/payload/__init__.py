"""Benchmark payloads: the two architectures the end-to-end configurations name.
They are plain nn.Modules with one module object per use (FX module swapping keys
its per-layer metadata by module path), random-initialised."""
from .resnet import resnet50  # noqa: F401
from .vit import vit_b16  # noqa: F401
