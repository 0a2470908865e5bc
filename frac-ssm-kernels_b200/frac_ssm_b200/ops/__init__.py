"""Scan ops: the dispatcher `frac_scan` and the per-stage forward ops of the b200 backend."""

from .b200.stages import (chunk_cumsum, chunk_fused_readout, chunk_readout, chunk_state, chunk_w,
                          state_passing)
from .frac_scan import cute_supported, frac_scan
from .registry import BACKENDS, IMPLS, available, load

__all__ = ["BACKENDS", "IMPLS", "available", "load", "cute_supported", "frac_scan", "chunk_cumsum",
           "chunk_state", "state_passing", "chunk_w", "chunk_readout", "chunk_fused_readout"]
