"""frac_ssm_b200 — the FRAC fractional-SSM chunked scan (forward) on NVIDIA B200 (sm_100a).

Host code is PyTorch over a C-ABI CUDA library (`lib/libfracssm.so`, declared in
`include/fracssm.h`).  The entry points keep the names and signatures of
quorbix/frac-ssm-kernels so its layers and models can call them unchanged.
"""

from .ops.frac_scan import cute_supported, frac_scan

__version__ = "0.1.0"

__all__ = ["__version__", "cute_supported", "frac_scan"]
