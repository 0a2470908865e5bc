"""Backend registry with the reference's interface (`frac_ssm/ops/registry.py:13-59`).

There is a single backend here, "b200": the sm_100a CUDA extension.  To use it from the
reference package, add `"b200": "frac_ssm_b200.ops.b200.frac_scan"` to its `IMPLS` table.
"""

from __future__ import annotations

import importlib
from types import ModuleType

BACKENDS = ("b200",)

IMPLS: dict[str, str] = {"b200": "frac_ssm_b200.ops.b200.frac_scan"}


def available(backend: str) -> tuple[bool, str | None]:
    """Whether this backend can run in the current environment."""
    _check_backend(backend)
    import os

    import torch

    from .. import _cabi

    if not os.path.exists(_cabi.lib_path()):
        return False, "libfracssm.so has not been built"
    if not torch.cuda.is_available():
        return False, "CUDA device required"
    cap = torch.cuda.get_device_capability()
    if cap[0] != 10:
        return False, f"Device with sm_100 cc is required, found sm_{cap[0]}{cap[1]}"
    return True, None


def load(backend: str | None = None) -> ModuleType:
    """Load a backend module; ``None`` picks "b200"."""
    if backend is None:
        backend = "b200"
    _check_backend(backend)
    ok, reason = available(backend)
    if not ok:
        raise RuntimeError(f"Backend {backend!r} is unavailable: {reason}")
    return importlib.import_module(IMPLS[backend])


def _check_backend(backend: str) -> None:
    if backend not in BACKENDS:
        raise ValueError(
            f"Unknown backend {backend!r}. Available backends: {', '.join(BACKENDS)}"
        )
