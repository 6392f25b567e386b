"""Puts the reference's Triton operator modules where the benchmark and the GPU parity test
can import them: `baseline/_ref/` (git-ignored, so the reference's sources never enter this
repository's history; the folder still travels with a working copy to the GPU machine).

    python baseline/install_reference.py /path/to/Deep_Optimization

Copied, unmodified: Activation_Compression/act_triton_kernel.py (the `act_lib::` codec
operators, lines 336-433) and Activation_Compression/triton_kernel/linear.py (Triton_Linear).
The reference has no package metadata, so there is nothing for pip to install.
"""
import os
import shutil
import sys

FILES = ("Activation_Compression/act_triton_kernel.py", "Activation_Compression/triton_kernel/linear.py")


def install(ref_root: str) -> str:
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    os.makedirs(dst, exist_ok=True)
    for rel in FILES:
        src = os.path.join(ref_root, rel)
        if not os.path.exists(src):
            raise SystemExit(f"not found: {src}")
        shutil.copyfile(src, os.path.join(dst, os.path.basename(rel)))
    return dst


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print("installed into", install(sys.argv[1]))
