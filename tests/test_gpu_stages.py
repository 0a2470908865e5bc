"""Parity of every stage op (through the C ABI) with the CPU oracle and the golden fixtures."""

import os

import pytest
import torch

from oracle import frac_oracle as O
from tests.helpers import TOL_BF16, TOL_F32, assert_ref_error, close, cuda

pytestmark = pytest.mark.gpu

GENS = ["random", "model_like"]


@pytest.fixture(scope="module")
def ops():
    from frac_ssm_b200 import ops as _ops
    ok, why = _ops.available("b200")
    assert ok, f"the b200 backend must be usable on a GPU box: {why}"
    return _ops


def _golden(golden_dir, name):
    return torch.load(os.path.join(golden_dir, name + ".pt"), weights_only=False)


@pytest.mark.parametrize("gen", GENS)
@pytest.mark.parametrize("B,L,M,T", [(1, 1, 8, 16), (3, 70, 8, 16), (2, 4001, 16, 64),
                                     (17, 512, 128, 256), (2, 1000, 48, 128), (1, 2048, 5, 1024),
                                     (2, 700, 200, 256), (1, 300, 132, 32)])
def test_chunk_cumsum(ops, gen, B, L, M, T):
    lr = O.LOG_RHO_GENS[gen](B, L, M, seed=1)
    lcr, cd = ops.chunk_cumsum(lr.cuda(), T)
    lcr_pt, cd_pt = O.chunk_cumsum(lr, T, exact=False)
    lcr_ref, cd_ref = O.chunk_cumsum(lr, T, exact=True)
    close(lcr, lcr_pt, **TOL_F32)
    close(cd, cd_pt, **TOL_F32)
    assert_ref_error(lcr, lcr_pt, lcr_ref, 1e-4 * max(1.0, lcr_ref.abs().max().item()))
    assert_ref_error(cd, cd_pt, cd_ref, 1e-4 * max(1.0, cd_ref.abs().max().item()))


def test_chunk_cumsum_reconstructs_full_sum(ops):
    B, L, M, T = 2, 1000, 16, 64
    lr = O.model_like_log_rho(B, L, M, seed=7)
    lcr, cd = ops.chunk_cumsum(lr.cuda(), T)
    full = lr.double().cumsum(1)
    offs = torch.cat([torch.zeros(B, 1, M, dtype=torch.float64), cd.double().cpu().cumsum(1)[:, :-1]], 1)
    rebuilt = lcr.double().cpu() + offs.repeat_interleave(T, dim=1)[:, :L]
    torch.testing.assert_close(rebuilt, full, rtol=1e-4, atol=1e-3)


def test_chunk_cumsum_noncontiguous_rows(ops):
    base = O.uniform_log_rho(2, 100, 24, seed=3).cuda()
    view = base[:, :, :16]          # padded row stride
    lcr, cd = ops.chunk_cumsum(view, 32)
    lcr_pt, cd_pt = O.chunk_cumsum(view.cpu().contiguous(), 32)
    close(lcr, lcr_pt, **TOL_F32)
    close(cd, cd_pt, **TOL_F32)


def test_chunk_cumsum_unaligned_view(ops):
    """A source that starts 4 bytes off a 16-byte boundary takes the element-wise kernel."""
    base = O.uniform_log_rho(2, 100, 20, seed=5).cuda()
    view = base[:, :, 1:17]
    lcr, cd = ops.chunk_cumsum(view, 32)
    lcr_pt, cd_pt = O.chunk_cumsum(view.cpu().contiguous(), 32)
    close(lcr, lcr_pt, **TOL_F32)
    close(cd, cd_pt, **TOL_F32)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("gen", GENS)
@pytest.mark.parametrize("B,L,R,M,T", [(2, 1, 64, 16, 64), (3, 70, 8, 8, 16), (2, 1000, 64, 128, 256),
                                       (1, 512, 192, 16, 128), (2, 300, 40, 24, 64)])
def test_chunk_state(ops, dtype, gen, B, L, R, M, T):
    u, c, kappa, rho, _ = O.scan_inputs(B, L, R, M, dtype=dtype, gen=gen, seed=2)
    lcr, _ = O.chunk_cumsum(O.log_decay(rho), T)
    st = ops.chunk_state(u.cuda(), kappa.cuda(), lcr.cuda(), T, state_fp32=True)
    st_pt = O.chunk_state(u, kappa, lcr, T, state_fp32=True, exact=False)
    st_ref = O.chunk_state(u.float(), kappa.float(), lcr, T, state_fp32=True, exact=True)
    assert st.dtype == torch.float32
    close(st, st_ref, **TOL_F32)
    assert_ref_error(st, st_pt, st_ref, 1e-4)
    if dtype == torch.bfloat16:
        st16 = ops.chunk_state(u.cuda(), kappa.cuda(), lcr.cuda(), T, state_fp32=False)
        assert st16.dtype == torch.bfloat16
        close(st16, st_ref, **TOL_BF16)


@pytest.mark.parametrize("sdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("with_init", [False, True])
@pytest.mark.parametrize("B,N,R,M", [(2, 1, 8, 8), (3, 17, 64, 16), (2, 32, 64, 128)])
def test_state_passing(ops, sdtype, with_init, B, N, R, M):
    g = torch.Generator().manual_seed(11)
    states = (0.25 * torch.randn(B, N, R, M, generator=g)).to(sdtype)
    cd = -torch.rand(B, N, M, generator=g) * 3.0
    init = 0.25 * torch.randn(B, R, M, generator=g) if with_init else None
    acc, fin = ops.state_passing(states.cuda(), cd.cuda(), None if init is None else init.cuda())
    acc_pt, fin_pt = O.state_passing(states, cd, init, exact=False)
    acc_ref, fin_ref = O.state_passing(states.float(), cd, init, exact=True)
    assert acc.dtype == sdtype and fin.dtype == sdtype
    tol = TOL_F32 if sdtype == torch.float32 else TOL_BF16
    close(acc, acc_ref, **tol)
    close(fin, fin_ref, **tol)
    assert_ref_error(acc, acc_pt, acc_ref, 2e-4)
    assert_ref_error(fin, fin_pt, fin_ref, 2e-4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("gen", GENS)
@pytest.mark.parametrize("B,L,M,T", [(2, 1, 16, 32), (2, 200, 16, 64), (1, 300, 128, 256), (3, 96, 8, 32)])
def test_chunk_w(ops, dtype, gen, B, L, M, T):
    _, c, kappa, rho, _ = O.scan_inputs(B, L, 8, M, dtype=dtype, gen=gen, seed=4)
    lcr, _ = O.chunk_cumsum(O.log_decay(rho), T)
    W = ops.chunk_w(c.cuda(), kappa.cuda(), lcr.cuda(), T)
    W_pt = O.chunk_w(c, kappa, lcr, T, exact=False)
    W_ref = O.chunk_w(c.float(), kappa.float(), lcr, T, exact=True)
    close(W, W_ref, **TOL_F32)
    assert_ref_error(W, W_pt, W_ref, 1e-5)
    assert torch.equal(W.cpu().triu(1), torch.zeros_like(W_ref))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,L,R,M,T", [(2, 1, 64, 16, 64), (2, 200, 64, 16, 64), (1, 300, 64, 128, 256),
                                       (3, 70, 8, 8, 16), (1, 257, 192, 16, 128)])
def test_chunk_readout_and_fused(ops, dtype, B, L, R, M, T):
    u, c, kappa, rho, init = O.scan_inputs(B, L, R, M, dtype=dtype, gen="model_like", seed=5)
    lcr, cd = O.chunk_cumsum(O.log_decay(rho), T)
    st = O.chunk_state(u.float(), kappa.float(), lcr, T, exact=True)
    acc, _ = O.state_passing(st, cd, init, exact=True)
    acc = acc.float()
    W = O.chunk_w(c.float(), kappa.float(), lcr, T, exact=True)
    h_ref = O.chunk_readout(u.float(), c.float(), acc, W, lcr, T, exact=True)
    h_pt = O.chunk_readout(u, c, acc, W, lcr, T, exact=False)
    tol = TOL_F32 if dtype == torch.float32 else TOL_BF16
    ug, cg, kg, ag, Wg, lg = cuda(u, c, kappa, acc, W, lcr)
    h = ops.chunk_readout(ug, cg, ag, Wg, lg, T)
    assert h.dtype == dtype
    close(h, h_ref, **tol)
    assert_ref_error(h, h_pt, h_ref, 1e-5 if dtype == torch.float32 else 2e-2)
    hf = ops.chunk_fused_readout(ug, cg, kg, ag, lg, T)
    close(hf, h_ref, **tol)
    assert_ref_error(hf, h_pt, h_ref, 1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("name", ["scan_f32_ragged", "scan_f32_random", "scan_bf16_init", "scan_bf16_ragged"])
def test_stages_on_golden_fixtures(ops, golden_dir, name):
    """Each CUDA stage on the fixture inputs against the outputs the reference produced."""
    g = _golden(golden_dir, name)
    T = g["meta"]["T"]
    u, c, kappa, rho, init = g["u"], g["c"], g["kappa"], g["rho"], g["initial_state"]
    ref = g["exact"]
    tol = TOL_F32 if u.dtype == torch.float32 else TOL_BF16
    ug, cg, kg, rg = cuda(u, c, kappa, rho)
    ig = None if init is None else init.cuda()
    lcr, cd = ops.chunk_cumsum(torch.log(rg.clamp(min=1e-6)), T)
    close(lcr, ref["lcr"], **TOL_F32)
    close(cd, ref["chunk_decay"], **TOL_F32)
    st = ops.chunk_state(ug, kg, lcr, T, state_fp32=True)
    close(st, ref["states"], **TOL_F32)
    acc, fin = ops.state_passing(st, cd, ig)
    close(acc, ref["states_acc"], **TOL_F32)
    close(fin, ref["final_state"], **TOL_F32)
    if T % 32 == 0 and c.shape[-1] & (c.shape[-1] - 1) == 0:
        W = ops.chunk_w(cg, kg, lcr, T)
        close(W, ref["W"], **TOL_F32)
        h = ops.chunk_readout(ug, cg, acc, W, lcr, T)
        close(h, ref["h"], **tol)
    hf = ops.chunk_fused_readout(ug, cg, kg, acc, lcr, T)
    close(hf, ref["h"], **tol)


def test_zero_batch_shapes(ops):
    z = torch.zeros(0, 64, 16, device="cuda")
    lcr, cd = ops.chunk_cumsum(z, 32)
    assert lcr.shape == (0, 64, 16) and cd.shape == (0, 2, 16)
    u = torch.zeros(0, 64, 8, device="cuda", dtype=torch.bfloat16)
    st = ops.chunk_state(u, z.bfloat16(), z, 32)
    assert st.shape == (0, 2, 8, 16)
    acc, fin = ops.state_passing(st, cd)
    assert acc.shape == (0, 2, 8, 16) and fin.shape == (0, 8, 16)
    assert ops.chunk_w(z, z, z, 32).shape == (0, 2, 32, 32)
    assert ops.chunk_fused_readout(u, z.bfloat16(), z.bfloat16(), acc, z, 32).shape == (0, 64, 8)


def test_stage_and_layer_ops_inside_torch_compile_fullgraph():
    """Every stage op, the layer ops and the gated norm are registered custom ops with shape-only
    implementations, so a graph around them compiles without breaks (the reference checks the same
    for its ops, tests/test_frac_scan.py:249-262)."""
    from frac_ssm_b200 import ops
    from frac_ssm_b200.layers import scan_epilogue, skip_mix
    from frac_ssm_b200.modules import rmsnorm_gated_fwd
    B, L, R, M, T, H = 4, 96, 64, 16, 32, 2
    u, c, kappa, rho, init = (t.cuda() for t in O.scan_inputs(B, L, R, M, dtype=torch.float32, gen="model_like", seed=2))
    g = torch.Generator().manual_seed(3)
    x = torch.randn(B // H, L, H * R, generator=g).cuda()
    z = torch.randn(B // H, L, H * R, generator=g).cuda()
    D = torch.randn(H, R, generator=g).cuda()
    w = torch.ones(H * R).cuda()

    def fn(u, c, kappa, rho, init, x, z):
        lcr, cd = ops.chunk_cumsum(torch.log(rho.clamp(min=1e-6)), T)
        st = ops.chunk_state(u, kappa, lcr, T)
        acc, fin = ops.state_passing(st, cd, init)
        W = ops.chunk_w(c, kappa, lcr, T)
        h1 = ops.chunk_readout(u, c, acc, W, lcr, T)
        h2 = ops.chunk_fused_readout(u, c, kappa, acc, lcr, T)
        mixed = skip_mix(h1, x, D, H, R)
        y1, _ = rmsnorm_gated_fwd(mixed, w, z, 1e-6)
        y2 = scan_epilogue(h2, x, z, D, w, H, R, 1e-6)
        return h1 + 0.0, y1 * 1.0, y2 * 1.0, fin + 0.0

    eager = fn(u, c, kappa, rho, init, x, z)
    compiled = torch.compile(fn, fullgraph=True)(u, c, kappa, rho, init, x, z)
    for a, b in zip(compiled, eager):
        torch.testing.assert_close(a, b)
