"""The allocation-free scan entry point against the regular one (collected last on purpose).

`fracssm_frac_scan_fwd_noalloc` serves callers that cannot hand the library scratch memory and
must not trigger an allocation (allocator callbacks, no-cudaMalloc serving loops, bindings with
no device allocator).  Its scratch is a fixed array inside the library, shared by every call, so
the test runs it twice in a row and checks both results against the workspace-based entry point
and against the CPU oracle.
"""

import pytest
import torch

from oracle import frac_oracle as O
from tests.helpers import TOL_BF16, TOL_F32

pytestmark = pytest.mark.gpu


def _noalloc(u, c, kappa, rho, init, h=None):
    from frac_ssm_b200 import _cabi as C
    B, L, R = u.shape
    M = c.shape[-1]
    h = torch.empty_like(u) if h is None else h
    fin = torch.empty(B, R, M, device=u.device, dtype=torch.float32)
    C.check(C.lib().fracssm_frac_scan_fwd_noalloc(
        C.ptr(u), C.ptr(c), C.ptr(kappa), C.ptr(rho), C.ptr(init), C.ptr(h), C.ptr(fin), C.F32,
        B, L, R, M, C.stream_of(u)), "frac_scan_fwd_noalloc")
    return h, fin


def test_noalloc_matches_workspace_entry_twice_in_a_row():
    from frac_ssm_b200 import _cabi as C
    from frac_ssm_b200.ops.b200 import frac_scan
    cases = [O.scan_inputs(7, 700, 64, 128, gen="model_like", seed=31),
             O.scan_inputs(64, 300, 64, 128, gen="random", seed=32)]
    for use_init, case in zip((True, False), cases):
        u, c, kappa, rho, init = (t.cuda() for t in case)
        init = init if use_init else None
        h_ref, f_ref = frac_scan(u, c, kappa, rho, 256, init, True, final_state_dtype=torch.float32,
                                 path="fused", check=True)
        uc, cc, kc, rc, _ = case
        h_orc, f_orc = O.frac_scan_slabs(uc.float(), cc.float(), kc.float(), rc, 256,
                                         case[4] if use_init else None, True, exact=True, slab=8)
        for _ in range(2):
            h, fin = _noalloc(u, c, kappa, rho, init)
            assert C.lib().fracssm_frac_scan_noalloc_status(C.stream_of(u)) == 0     # synchronises
            torch.testing.assert_close(h.float(), h_ref.float(), **TOL_BF16)
            torch.testing.assert_close(fin, f_ref, **TOL_F32)
            torch.testing.assert_close(h.float().cpu(), h_orc.float(), **TOL_BF16)
            torch.testing.assert_close(fin.cpu(), f_orc.float(), **TOL_F32)


def test_output_rows_that_are_only_16_byte_aligned():
    """The kernel writes a row's 32 bytes per lane with one store when h is 32-byte aligned and with two
    16-byte stores otherwise: both give the same bits."""
    from frac_ssm_b200 import _cabi as C
    u, c, kappa, rho, _ = (t.cuda() for t in O.scan_inputs(5, 333, 64, 128, gen="model_like", seed=33))
    h_even, f_even = _noalloc(u, c, kappa, rho, None)
    assert C.ptr(h_even).value % 32 == 0
    buf = torch.full((u.numel() + 16,), float("nan"), device=u.device, dtype=u.dtype)
    h_odd = buf[8:8 + u.numel()].view_as(u)
    assert C.ptr(h_odd).value % 32 == 16
    h_odd, f_odd = _noalloc(u, c, kappa, rho, None, h=h_odd)
    assert C.lib().fracssm_frac_scan_noalloc_status(C.stream_of(u)) == 0
    assert torch.equal(h_odd, h_even) and torch.equal(f_odd, f_even)
    assert torch.isnan(buf[:8]).all() and torch.isnan(buf[8 + u.numel():]).all()


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from frac_ssm_b200 import _cabi as C
    u, c, kappa, rho, _ = (t.cuda() for t in O.scan_inputs(65, 128, 64, 128, seed=1))
    with pytest.raises(C.FracSsmError, match="exceeds the built-in scratch"):
        _noalloc(u, c, kappa, rho, None)
    u, c, kappa, rho, _ = (t.cuda() for t in O.scan_inputs(2, 128, 64, 64, seed=1))
    with pytest.raises(C.FracSsmError, match="R = 64, M = 128"):
        _noalloc(u, c, kappa, rho, None)
