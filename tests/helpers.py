"""Shared helpers for the GPU parity tests."""

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
