"""The tcgen05 / TMEM / TMA building blocks against a host matmul (one 128-row MMA tile)."""

import pytest
import torch

from tests.helpers import selftest_lib

pytestmark = pytest.mark.gpu


def _run(a_mn, b_mn, N, group0=0, sbo=1024, tma=False, seed=0):
    from frac_ssm_b200 import _cabi as C
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(128, 128, generator=g).bfloat16().float()
    B = torch.randn(128, 128, generator=g).bfloat16().float()
    Ad, Bd = A.cuda(), B.cuda()
    B16 = B[:, :64].contiguous().bfloat16().cuda()
    D = torch.full((128, N), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    C.check(selftest_lib().fracssm_selftest_umma(C.ptr(Ad), C.ptr(Bd), C.ptr(B16), C.ptr(D), C.ptr(status),
                                          int(a_mn), int(b_mn), N, group0, sbo, int(tma),
                                          C.stream_of(Ad)), "selftest_umma")
    torch.cuda.synchronize()
    assert status.item() == 0, "the MMA completion wait timed out"
    Am = A.t() if a_mn else A                     # [M, K]
    if b_mn:
        Bm = B[:, :N].t()                         # rows are k, columns n -> [N, K]
    else:
        rows = torch.cat([torch.arange(8) + 8 * (group0 + i * (sbo // 1024)) for i in range(N // 8)])
        Bm = B[rows]                              # [N, K]
    ref = Am @ Bm.t()
    torch.testing.assert_close(D.cpu(), ref, rtol=1e-4, atol=1e-3)


def test_k_major_both():
    _run(False, False, 128)


def test_k_major_b_strided_row_groups():
    _run(False, False, 64, group0=0, sbo=2048)     # every other 8-row group
    _run(False, False, 32, group0=1, sbo=4096)     # groups 1, 5, 9, 13
    _run(False, False, 32, group0=8, sbo=1024)     # rows 64..95
    _run(False, False, 64, group0=0, sbo=1024)


def test_mn_major_b():
    _run(False, True, 64)


def test_mn_major_b_two_atoms():
    _run(False, True, 128)                         # 128 columns = two 64-wide atoms side by side


def test_mn_major_a_and_b():
    _run(True, True, 64)


def test_mn_major_b_via_tma():
    _run(False, True, 64, tma=True)
    _run(True, True, 64, tma=True, seed=3)


def test_64_row_mma_lane_layout():
    """A 64-row MMA puts result rows 16q..16q+15 into tensor-memory lanes 32q..32q+15."""
    from frac_ssm_b200 import _cabi as C
    g = torch.Generator().manual_seed(3)
    A = torch.randn(128, 128, generator=g).bfloat16().float()
    B = torch.randn(128, 128, generator=g).bfloat16().float()
    Ad, Bd = A.cuda(), B.cuda()
    for N in (64, 16):
        D = torch.full((128, N), -777.0, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        C.check(selftest_lib().fracssm_selftest_umma_m64(C.ptr(Ad), C.ptr(Bd), C.ptr(D), C.ptr(status), N,
                                                  C.stream_of(Ad)), "selftest_umma_m64")
        torch.cuda.synchronize()
        assert status.item() == 0, "the MMA completion wait timed out"
        ref = A[:64] @ B[:N].t()
        lanes = torch.cat([torch.arange(16) + 32 * q for q in range(4)])
        torch.testing.assert_close(D.cpu()[lanes], ref, rtol=1e-4, atol=1e-3)
