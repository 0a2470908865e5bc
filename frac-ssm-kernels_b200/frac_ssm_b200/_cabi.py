"""ctypes binding of libfracssm.so (the C ABI declared in include/fracssm.h).

There is no fallback: if the shared library is missing the import of any op raises, and
every call checks the returned status and raises with the library's error text.
"""

from __future__ import annotations

import contextlib
import ctypes
import os
import threading

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libfracssm.so")
_lock = threading.Lock()
_lib = None

F32, BF16, F16 = 0, 1, 2
_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

PATH_AUTO, PATH_STAGED, PATH_FUSED = 0, 1, 2
ABI_VERSION = 2       # FRACSSM_ABI_VERSION of include/fracssm.h this binding was written against

i64, ci, cf, vp, sz = ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t

_SIGNATURES = {
    "fracssm_abi_version": (ci, []),
    "fracssm_last_error": (ctypes.c_char_p, []),
    "fracssm_scan_fused_supported": (ci, [i64, i64, i64, i64, i64, ci, ci]),
    "fracssm_chunk_cumsum": (ci, [vp, i64, i64, ci, vp, vp, i64, i64, i64, i64, vp]),
    "fracssm_chunk_state": (ci, [vp, ci, i64, i64, vp, ci, i64, i64, vp, i64, i64, vp, ci,
                                 i64, i64, i64, i64, i64, vp]),
    "fracssm_state_passing": (ci, [vp, ci, vp, vp, ci, vp, ci, vp, ci, i64, i64, i64, i64, vp]),
    "fracssm_chunk_w": (ci, [vp, vp, ci, i64, i64, i64, i64, vp, i64, i64, vp, i64, i64, i64, i64, vp]),
    "fracssm_chunk_readout": (ci, [vp, ci, i64, i64, vp, ci, i64, i64, vp, ci, vp, ci, vp, i64, i64,
                                   vp, i64, i64, i64, i64, i64, vp]),
    "fracssm_chunk_fused_readout": (ci, [vp, ci, i64, i64, vp, vp, ci, i64, i64, i64, i64, vp, ci,
                                         vp, i64, i64, vp, i64, i64, i64, i64, i64, vp]),
    "fracssm_frac_scan_workspace_bytes": (sz, [i64, i64, i64, i64, i64, ci]),
    "fracssm_frac_scan_fwd": (ci, [vp, ci, i64, i64, vp, vp, ci, i64, i64, i64, i64, vp, i64, i64,
                                   vp, vp, vp, ci, vp, sz, i64, i64, i64, i64, i64, ci, vp]),
    "fracssm_frac_scan_fwd_noalloc": (ci, [vp, vp, vp, vp, vp, vp, vp, ci, i64, i64, i64, i64, vp]),
    "fracssm_segment_summary_workspace_bytes": (sz, [i64, i64, i64]),
    "fracssm_segment_summary": (ci, [vp, vp, ci, vp, vp, vp, vp, vp, sz, i64, i64, i64, i64, vp]),
    "fracssm_segment_summary_grouped": (ci, [vp, vp, ci, vp, vp, vp, vp, sz, i64, i64, i64, i64, i64, vp]),
    "fracssm_scan_fused_status": (ci, [vp, vp]),
    "fracssm_frac_scan_noalloc_status": (ci, [vp]),
    "fracssm_compute_params": (ci, [vp, ci, i64, i64, vp, ci, i64, i64, vp, ci, i64, i64,
                                    vp, i64, i64, vp, vp, vp, vp, cf, cf, cf, cf, cf, cf, cf,
                                    vp, vp, vp, ci, vp, i64, i64, i64, i64, i64, vp]),
    "fracssm_skip_mix": (ci, [vp, ci, i64, i64, vp, ci, i64, i64, vp, vp, ci, i64, i64, i64, i64, vp]),
    "fracssm_rmsnorm_gated": (ci, [vp, i64, vp, i64, ci, vp, ci, cf, vp, vp, i64, i64, vp]),
    "fracssm_scan_epilogue": (ci, [vp, ci, i64, i64, vp, i64, i64, vp, i64, i64, ci, vp, vp, ci,
                                   cf, cf, vp, i64, i64, i64, i64, vp]),
    "fracssm_scan_layer_workspace_bytes": (sz, [i64, i64, i64, i64, i64]),
    "fracssm_scan_layer_gated": (ci, [vp, vp, vp, ci, vp, vp, vp, vp, cf, vp, vp, vp, ci, vp, sz,
                                      i64, i64, i64, i64, i64, vp]),
    "fracssm_scan_layer_sumsq": (ci, [vp, vp, i64, i64, i64, vp]),
    "fracssm_scan_layer_norm": (ci, [vp, vp, vp, vp, ci, cf, i64, vp, i64, i64, i64, i64, vp]),
    "fracssm_causal_conv_silu": (ci, [vp, ci, i64, i64, vp, i64, i64, vp, vp, ci, vp, ci, i64, i64, i64,
                                      i64, vp]),
    "fracssm_causal_conv_silu_heads": (ci, [vp, ci, i64, i64, vp, i64, i64, vp, vp, ci, vp, ci, vp, i64, i64, i64,
                                            i64, i64, vp]),
    "fracssm_decode_step": (ci, [vp, ci, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, vp]),
    "fracssm_scan_epilogue_sumsq": (ci, [vp, ci, i64, i64, vp, i64, i64, vp, i64, i64, ci, vp, cf, vp,
                                         i64, i64, i64, i64, vp]),
    "fracssm_scan_epilogue_apply": (ci, [vp, ci, i64, i64, vp, i64, i64, vp, i64, i64, ci, vp, vp, ci,
                                         cf, cf, vp, i64, vp, i64, i64, i64, i64, vp]),
}


class FracSsmError(RuntimeError):
    """A libfracssm.so call returned a non-zero status."""


def lib_path() -> str:
    return _LIB_PATH


def lib():
    """Load (once) and return the shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(_LIB_PATH):
                    raise ImportError(
                        f"{_LIB_PATH} is missing: build it with "
                        "`python frac-ssm-kernels_b200/build.py` (needs nvcc). "
                        "There is no CPU fallback.")
                handle = ctypes.CDLL(_LIB_PATH)
                for name, (res, args) in _SIGNATURES.items():
                    fn = getattr(handle, name)
                    fn.restype, fn.argtypes = res, args
                if handle.fracssm_abi_version() != ABI_VERSION:
                    raise ImportError("libfracssm.so has an unexpected ABI version")
                _lib = handle
    return _lib


def dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise AssertionError(f"unsupported dtype {t.dtype}") from None


def dt_of(dtype: torch.dtype) -> int:
    return _DT[dtype]


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_of(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def rows(t: torch.Tensor) -> torch.Tensor:
    """Return t with a unit stride on its last dim (copy only if needed)."""
    return t if t.stride(-1) == 1 else t.contiguous()


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().fracssm_last_error().decode("utf-8", "replace")
        raise FracSsmError(f"{what} failed (status {status}): {msg}")


_NVTX = os.environ.get("FRACSSM_NVTX", "") not in ("", "0")


def trace(name: str):
    """NVTX range around a host-side stage when FRACSSM_NVTX=1 (for nsys / ncu timelines; the
    reference marks its stages the same way, `frac_ssm/ops/utils.py:6-23`); a no-op otherwise."""
    if not _NVTX:
        return contextlib.nullcontext()
    return torch.cuda.nvtx.range(name)
