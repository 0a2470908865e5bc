"""The sm_100a backend: stage ops and the composed scan."""

from .frac_scan import frac_scan
from .stages import (chunk_cumsum, chunk_fused_readout, chunk_readout, chunk_state, chunk_w,
                     state_passing)

__all__ = ["frac_scan", "chunk_cumsum", "chunk_state", "state_passing", "chunk_w", "chunk_readout",
           "chunk_fused_readout"]
