"""Shared helpers for the GPU parity tests."""

import ctypes
import os

import torch

from oracle import frac_oracle as O

# Tolerances of the acceptance criteria: float32 cumsums/states within rtol = atol = 1e-3 of the
# float32 reference; bfloat16 outputs within 2e-2.
TOL_F32 = dict(rtol=1e-3, atol=1e-3)
TOL_BF16 = dict(rtol=2e-2, atol=2e-2)


def assert_ref_error(out, out_pt, out_ref, atol):
    """The reference suite's three-way rule (its tests/test_frac_scan.py:37-41): the kernel may be
    at most twice as far from the float64-decay truth as the working-precision reference is."""
    assert out.shape == out_ref.shape
    err = (out.float().cpu() - out_ref.float()).abs().max().item()
    err_pt = (out_pt.float() - out_ref.float()).abs().max().item()
    assert err <= 2 * err_pt + atol, f"error {err:.3e} > 2 * {err_pt:.3e} + {atol}"


def close(out, ref, **tol):
    torch.testing.assert_close(out.float().cpu(), ref.float(), **tol)


def scan_case(B, L, R, M, dtype, gen, seed=0):
    return O.scan_inputs(B, L, R, M, dtype=dtype, gen=gen, seed=seed)


def cuda(*ts):
    return tuple(None if t is None else t.cuda() for t in ts)


_SELFTEST = None


def selftest_lib():
    """The test-only library (include/fracssm_selftest.h): the product sources plus csrc/selftest."""
    global _SELFTEST
    if _SELFTEST is None:
        from frac_ssm_b200 import _cabi as C
        path = os.path.join(os.path.dirname(C.lib_path()), "libfracssm_selftest.so")
        h = ctypes.CDLL(path)
        vp, ci, i64, sz, u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t, ctypes.c_uint64
        h.fracssm_last_error.restype = ctypes.c_char_p
        sigs = {
            "fracssm_selftest_umma": [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp],
            "fracssm_selftest_umma_m64": [vp, vp, vp, vp, ci, vp],
            "fracssm_selftest_scan_wait_limit": [vp, vp, vp, vp, vp, vp, vp, sz, i64, i64, u64, vp],
            "fracssm_selftest_summary_wait_limit": [vp, vp, vp, vp, vp, vp, sz, i64, i64, u64, vp],
            "fracssm_scan_fused_status": [vp, vp],
            "fracssm_frac_scan_workspace_bytes": [i64, i64, i64, i64, i64, ci],
            "fracssm_segment_summary_workspace_bytes": [i64, i64, i64],
        }
        for name, args in sigs.items():
            fn = getattr(h, name)
            fn.argtypes = args
            fn.restype = sz if name.endswith("workspace_bytes") else ci
        _SELFTEST = h
    return _SELFTEST
