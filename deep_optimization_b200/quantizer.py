"""Bit-allocation policy (Activation_Compression/quantizer.py:13-127).

Only the parts on the compression path are here: the per-target bit table, the
default-bits assignment, the tensor filter and the Hessian-eigenvalue lookup
table.  The reference's research probes (Hessian power iteration, Lanczos
density, low-rank and low-frequency-energy analyses) are not part of this path.
`check_quantize` tests the rank with `len(t.shape)` (the reference calls `len` on
a boolean there).
"""
from __future__ import annotations

import torch


class Quantizer:
    def __init__(self, config, target_dict):
        self.unrelated_tensors = set()
        self.default_bit = config["default_bits"]
        self.config = config
        self.bits = target_dict
        self.dims = {}
        self.graph_mode = False

    def filter_tensors(self, pair):
        for _, v in pair:
            self.unrelated_tensors.add(v.data_ptr())

    def check_quantize(self, input_tensor: torch.Tensor) -> bool:
        if input_tensor.data_ptr() in self.unrelated_tensors:
            return False
        if input_tensor.dtype not in (torch.float16, torch.float32, torch.bfloat16):
            return False
        if not input_tensor.requires_grad:
            return False
        return input_tensor.dim() in (2, 3, 4)

    def clean_iterate(self):
        self.bits.clear()
        self.dims.clear()

    def iterate(self, model=None, criterion=None, dataloader=None):
        """Every registered target gets `default_bits` (quantizer.py:51-56); the
        auto-precision branch of the reference is an unfinished experiment."""
        if self.config.get("auto_precision") is not None:
            raise NotImplementedError("auto_precision probes are outside the compression path")
        for target in list(self.bits):
            self.bits[target] = self.config["default_bits"]

    @staticmethod
    def hessian2bit_lookup_table(eigenvalue: float) -> int:
        """quantizer.py:117-127"""
        if eigenvalue >= 1000:
            return 8
        if eigenvalue >= 500:
            return 4
        if eigenvalue >= 250:
            return 3
        if eigenvalue >= 50:
            return 2
        return 1
