"""A bounded device-side wait that runs out: the kernels return by themselves, the status call
reports FRACSSM_ERR_WAIT and the outputs are marked with NaN.  Nothing here faults or hangs the GPU:
the launch simply starts at the second tile of every row, whose predecessor is not part of it, with a
wait limit of a few milliseconds (include/fracssm_selftest.h)."""

import ctypes
import time

import pytest
import torch

from oracle import frac_oracle as O
from tests.helpers import selftest_lib

pytestmark = pytest.mark.gpu

ERR_WAIT = 4


def _ws(nbytes):
    return torch.zeros(max(int(nbytes), 256), dtype=torch.uint8, device="cuda")


def test_scan_wait_runs_out_and_is_reported():
    from frac_ssm_b200 import _cabi as C
    lib = selftest_lib()
    B, L = 3, 384
    u, c, kappa, rho, _ = (t.cuda() for t in O.scan_inputs(B, L, 64, 128, gen="model_like", seed=11))
    h = torch.zeros_like(u)
    fin = torch.zeros(B, 64, 128, device="cuda")
    ws = _ws(lib.fracssm_frac_scan_workspace_bytes(B, L, 64, 128, 128, 2))
    stream = C.stream_of(u)
    t0 = time.time()
    rc = lib.fracssm_selftest_scan_wait_limit(C.ptr(u), C.ptr(c), C.ptr(kappa), C.ptr(rho), C.ptr(h), C.ptr(fin),
                                              C.ptr(ws), ws.numel(), B, L, ctypes.c_uint64(2_000_000), stream)
    assert rc == 0, lib.fracssm_last_error()
    status = lib.fracssm_scan_fused_status(C.ptr(ws), stream)       # synchronises
    assert time.time() - t0 < 5.0, "the kernel did not return promptly after its wait limit"
    assert status == ERR_WAIT
    assert b"wait ran out" in lib.fracssm_last_error()
    assert torch.isnan(h[:, 128:].float()).all(), "outputs after a failed wait must be NaN"
    assert torch.isnan(fin).all()
    assert (h[:, :128] == 0).all(), "tokens outside the launch were touched"
    # the context is still usable and the regular entry point works afterwards
    from frac_ssm_b200.ops.b200 import frac_scan
    out = frac_scan(u, c, kappa, rho, 256, None, False, check=True)
    assert torch.isfinite(out.float()).all()


def test_summary_wait_runs_out_and_is_reported():
    from frac_ssm_b200 import _cabi as C
    lib = selftest_lib()
    B, L = 2, 256
    u, _, kappa, rho, _ = (t.cuda() for t in O.scan_inputs(B, L, 64, 128, gen="random", seed=12))
    fin = torch.zeros(B, 64, 128, device="cuda")
    dec = torch.zeros(B, 128, device="cuda")
    ws = _ws(lib.fracssm_segment_summary_workspace_bytes(B, 64, 128))
    stream = C.stream_of(u)
    rc = lib.fracssm_selftest_summary_wait_limit(C.ptr(u), C.ptr(kappa), C.ptr(rho), C.ptr(fin), C.ptr(dec),
                                                 C.ptr(ws), ws.numel(), B, L, ctypes.c_uint64(2_000_000), stream)
    assert rc == 0, lib.fracssm_last_error()
    assert lib.fracssm_scan_fused_status(C.ptr(ws), stream) == ERR_WAIT
    assert torch.isnan(fin).all() and torch.isnan(dec).all()
