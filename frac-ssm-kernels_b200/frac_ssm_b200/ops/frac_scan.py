"""Public fractional scan API: the reference's dispatcher signature
(`frac_ssm/ops/frac_scan.py:53-81`) over the single "b200" backend."""

from __future__ import annotations

import logging
import os

from .registry import available, load

_LOGGER = logging.getLogger(__name__)
_IMPL_ENV = "FRAC_SSM_IMPL"
_selection_logged = False


def cute_supported(*_args, **_kwargs) -> tuple[bool, str | None]:
    """The reference's Hopper CuTe backend does not exist in this package."""
    return False, "the sm_90 CuTe backend is not part of this package; use impl='b200'"


def frac_scan(u, c, kappa, rho, chunk_size, initial_state=None, return_final_state=False,
              cu_seqlens=None, impl=None):
    """Run the fractional scan.  Backend selection: ``impl`` > ``FRAC_SSM_IMPL`` > "b200".
    Variable-length sequences are not supported (as in the reference)."""
    global _selection_logged
    if cu_seqlens is not None:
        raise NotImplementedError("cu_seqlens is not supported yet")
    if impl is None:
        impl = os.environ.get(_IMPL_ENV)
    module = load(impl)
    if not _selection_logged:
        _LOGGER.info("Using frac_scan backend %r", impl or "b200")
        _selection_logged = True
    return module.frac_scan(u, c, kappa, rho, chunk_size, initial_state, return_final_state)


__all__ = ["available", "cute_supported", "frac_scan"]
