"""Parity of the composed scan (through the C ABI) with the CPU oracle, the golden fixtures
and size-independent properties."""

import os

import pytest
import torch

from oracle import frac_oracle as O
from tests.helpers import TOL_BF16, TOL_F32, assert_ref_error, close, cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def scan():
    from frac_ssm_b200 import ops
    ok, why = ops.available("b200")
    assert ok, f"the b200 backend must be usable on a GPU box: {why}"
    from frac_ssm_b200.ops.b200 import frac_scan
    return frac_scan


PATHS = ["staged", "auto"]


_REFS = {}


def _oracle(key, u, c, kappa, rho, T, init):
    """Oracle outputs, cached per test case so both kernel paths share one CPU evaluation."""
    if key not in _REFS:
        slab = max(1, min(u.shape[0], (1 << 27) // max(1, u.shape[1] * T * c.shape[-1])))
        ref = O.frac_scan_slabs(u.float(), c.float(), kappa.float(), rho, T, init, True,
                                exact=True, slab=slab)
        pt = O.frac_scan_slabs(u, c, kappa, rho, T, init, True, exact=False, slab=slab)
        if len(_REFS) > 4:
            _REFS.clear()
        _REFS[key] = (ref, pt)
    return _REFS[key]


def _check(scan, u, c, kappa, rho, T, init, path="auto", key=None):
    ug, cg, kg, rg = cuda(u, c, kappa, rho)
    ig = None if init is None else init.cuda()
    h, fin = scan(ug, cg, kg, rg, T, ig, True, final_state_dtype=torch.float32, path=path, check=True)
    key = key or (tuple(u.shape), c.shape[-1], T, u.dtype, c.dtype, init is None,
                  float(rho.double().sum()), float(u.double().sum()))
    (h_ref, fin_ref), (h_pt, fin_pt) = _oracle(key, u, c, kappa, rho, T, init)
    assert h.dtype == u.dtype and fin.dtype == torch.float32
    close(h, h_ref, **(TOL_F32 if u.dtype == torch.float32 else TOL_BF16))
    close(fin, fin_ref, **TOL_F32)
    assert_ref_error(h, h_pt, h_ref, 1e-4 if u.dtype == torch.float32 else 2e-2)
    assert_ref_error(fin, fin_pt, fin_ref, 1e-4)
    return h, fin


@pytest.mark.parametrize("path", PATHS)        # top decorator varies fastest: cache hits
@pytest.mark.parametrize("gen", ["random", "model_like"])
@pytest.mark.parametrize("with_init", [False, True])
@pytest.mark.parametrize("B,L,R,M,T", [
    (1, 1, 64, 16, 64), (17, 32, 64, 16, 64), (2, 4001, 64, 16, 128), (1, 4096, 128, 16, 64),
    (3, 1000, 64, 128, 256), (2, 2048, 64, 128, 256), (2, 700, 192, 16, 128), (2, 515, 64, 64, 64),
    (5, 129, 64, 128, 64), (1, 128, 64, 128, 128), (300, 257, 64, 128, 256), (2, 4096, 64, 128, 256),
])
def test_scan_bf16(scan, path, gen, with_init, B, L, R, M, T):
    u, c, kappa, rho, init = O.scan_inputs(B, L, R, M, dtype=torch.bfloat16, gen=gen, seed=0)
    _check(scan, u, c, kappa, rho, T, init if with_init else None, path)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("B,L,R,M,T", [(2, 300, 64, 16, 64), (1, 1024, 64, 64, 64), (2, 70, 8, 8, 16)])
def test_scan_f32(scan, path, B, L, R, M, T):
    u, c, kappa, rho, init = O.scan_inputs(B, L, R, M, dtype=torch.float32, gen="model_like", seed=3)
    _check(scan, u, c, kappa, rho, T, init, path)


@pytest.mark.parametrize("path", PATHS)
def test_scan_bf16_u_with_f32_coefficients(scan, path):
    # the model's prep emits float32 c/kappa for a bfloat16 u
    u, c, kappa, rho, init = O.scan_inputs(2, 600, 64, 128, dtype=torch.float32, gen="model_like", seed=9)
    _check(scan, u.bfloat16(), c, kappa, rho, 256, init, path)


@pytest.mark.parametrize("path", PATHS)
def test_scan_m8(scan, path):
    u, c, kappa, rho, init = O.scan_inputs(4, 257, 64, 8, dtype=torch.bfloat16, gen="random", seed=4)
    _check(scan, u, c, kappa, rho, 64, None, path)


@pytest.mark.parametrize("path", PATHS)
def test_config0(scan, golden_dir, path):
    """BASELINE config 0 against the reference's stored (subsampled) output."""
    g = torch.load(os.path.join(golden_dir, "config0_subsample.pt"), weights_only=False)
    d = O.layer_inputs(1, 1024, 8, 64, 64, G=1, seed=0, dtype=torch.float32)
    h, fin = scan(*cuda(d["u"], d["c"], d["kappa"], d["rho"]), 64, None, True, path=path)
    close(h[:, ::37, ::5], g["exact"]["h_sub"], **TOL_F32)
    close(fin[:, ::3, ::7], g["exact"]["final_sub"], **TOL_F32)


@pytest.mark.parametrize("name", ["scan_f32_ragged", "scan_f32_random", "scan_bf16_init", "scan_bf16_ragged"])
def test_scan_on_golden_fixtures(scan, golden_dir, name):
    g = torch.load(os.path.join(golden_dir, name + ".pt"), weights_only=False)
    T = g["meta"]["T"]
    u, c, kappa, rho, init = g["u"], g["c"], g["kappa"], g["rho"], g["initial_state"]
    ig = None if init is None else init.cuda()
    h, fin = scan(*cuda(u, c, kappa, rho), T, ig, True, final_state_dtype=torch.float32)
    close(h, g["exact"]["h"], **(TOL_F32 if u.dtype == torch.float32 else TOL_BF16))
    close(fin, g["exact"]["final_state"], **TOL_F32)
    # default state dtype follows the reference: bfloat16 when u is bfloat16
    _, fin2 = scan(*cuda(u, c, kappa, rho), T, ig, True)
    assert fin2.dtype == (torch.bfloat16 if u.dtype == torch.bfloat16 else torch.float32)
    assert scan(*cuda(u, c, kappa, rho), T, ig, False).shape == u.shape


@pytest.mark.parametrize("path", PATHS)
def test_masked_span_crossing_chunks(scan, path):
    # kappa = 0, rho = 1 over a span leaves the state untouched (the reference's mask identity)
    u, c, kappa, rho, _ = O.scan_inputs(2, 512, 64, 128, dtype=torch.bfloat16, gen="model_like", seed=6)
    kappa[:, 200:330] = 0
    rho[:, 200:330] = 1.0
    _check(scan, u, c, kappa, rho, 256, None, path)


@pytest.mark.parametrize("path", PATHS)
def test_noncontiguous_inputs(scan, path):
    B, L, R, M, T = 2, 300, 64, 128, 256
    u, c, kappa, rho, init = O.scan_inputs(B, L, R + 8, M + 16, dtype=torch.bfloat16, gen="random", seed=8)
    ug, cg, kg, rg = cuda(u, c, kappa, rho)
    uv, cv, kv, rv = ug[:, :, :R], cg[:, :, :M], kg[:, :, :M], rg[:, :, :M]
    h, fin = scan(uv, cv, kv, rv, T, None, True, final_state_dtype=torch.float32, path=path)
    h_ref, fin_ref = O.frac_scan(u[:, :, :R].float(), c[:, :, :M].float(), kappa[:, :, :M].float(),
                                 rho[:, :, :M].contiguous(), T, None, True, exact=True)
    close(h, h_ref, **TOL_BF16)
    close(fin, fin_ref, **TOL_F32)


def test_zero_batch_and_determinism(scan):
    u = torch.zeros(0, 64, 64, device="cuda", dtype=torch.bfloat16)
    m = torch.zeros(0, 64, 128, device="cuda", dtype=torch.bfloat16)
    h, fin = scan(u, m, m, m.float(), 64, None, True)
    assert h.shape == (0, 64, 64) and fin.shape == (0, 64, 128)
    u, c, kappa, rho, init = cuda(*O.scan_inputs(5, 1000, 64, 128, gen="model_like", seed=12))
    a = scan(u, c, kappa, rho, 256, init, True)
    b = scan(u, c, kappa, rho, 256, init, True)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])     # no atomics in the forward
    # no token at all: the initial state passes through, in the default (bf16) and the f32 state type
    h0, fin0 = scan(u[:, :0], c[:, :0], kappa[:, :0], rho[:, :0], 256, init, True)
    assert h0.shape == (5, 0, 64) and fin0.dtype == torch.bfloat16 and torch.equal(fin0, init.bfloat16())
    _, fin1 = scan(u[:, :0], c[:, :0], kappa[:, :0], rho[:, :0], 256, None, True)
    assert torch.count_nonzero(fin1) == 0


# ---- size-independent properties at the benchmark's full shape ---------------------------------

def _full_inputs(B=192, L=8192, R=64, M=128, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    u = (0.25 * torch.randn(B, L, R, device="cuda", generator=g)).bfloat16()
    c = (0.25 * torch.randn(B, L, M, device="cuda", generator=g)).bfloat16()
    kappa = (0.25 * torch.randn(B, L, M, device="cuda", generator=g)).bfloat16()
    tau = torch.linspace(0.0, 11.09, M, device="cuda").exp()
    dt = torch.nn.functional.softplus(torch.randn(B, L, 1, device="cuda", generator=g) - 1.0)
    rate = (0.25 + 3.75 * torch.rand(B, L, 1, device="cuda", generator=g)) ** (
        1.0 / (0.2 + 0.75 * torch.rand(B, L, 1, device="cuda", generator=g)))
    rho = torch.exp(-dt * rate / tau).clamp(1e-6, 1 - 1e-6)
    return u, c, kappa, rho


def test_full_size_split_and_slab_properties(scan):
    """Benchmark shape (batch 8 x 24 heads, L 8192, R 64, M 128, T 256):
    (1) scanning two halves with the state handed over equals scanning the whole,
    (2) two (batch, head) rows agree with the CPU oracle,
    (3) the final state equals the token recurrence's on one row."""
    u, c, kappa, rho = _full_inputs()
    T = 256
    h, fin = scan(u, c, kappa, rho, T, None, True, final_state_dtype=torch.float32, check=True)
    half = u.shape[1] // 2
    h1, f1 = scan(u[:, :half], c[:, :half], kappa[:, :half], rho[:, :half], T, None, True,
                  final_state_dtype=torch.float32)
    h2, f2 = scan(u[:, half:], c[:, half:], kappa[:, half:], rho[:, half:], T, f1, True,
                  final_state_dtype=torch.float32)
    torch.testing.assert_close(torch.cat([h1, h2], 1).float(), h.float(), **TOL_BF16)
    torch.testing.assert_close(f2, fin, **TOL_F32)
    for row in (0, 191):
        sl = slice(row, row + 1)
        uc, cc, kc, rc = u[sl].cpu(), c[sl].cpu(), kappa[sl].cpu(), rho[sl].cpu()
        h_ref, f_ref = O.frac_scan(uc.float(), cc.float(), kc.float(), rc, T, None, True, exact=True)
        close(h[sl], h_ref, **TOL_BF16)
        close(fin[sl], f_ref, **TOL_F32)
    _, f_tok = O.token_recurrence(u[5:6, :].cpu(), c[5:6].cpu(), kappa[5:6].cpu(), rho[5:6].cpu())
    close(fin[5:6], f_tok.float(), **TOL_F32)


def test_full_size_linearity(scan):
    u, c, kappa, rho = _full_inputs(B=48, seed=1)
    # quantise u to multiples of 1/32 below 2 so that u + u2 is exact in bfloat16: what is left
    # is the rounding of the three outputs (about 1.5 bfloat16 ulps, 2^-8 relative each)
    u = (u.float().clamp(-1.9, 1.9) * 32).round().div(32).bfloat16()
    u2 = torch.roll(u, 1, dims=0)
    ha = scan(u, c, kappa, rho, 256).float()
    hb = scan(u2, c, kappa, rho, 256).float()
    hs = scan((u.float() + u2.float()).bfloat16(), c, kappa, rho, 256).float()
    scale = max(1.0, ha.abs().max().item(), hb.abs().max().item())
    torch.testing.assert_close(hs, ha + hb, rtol=2e-2, atol=2e-2 * scale)


def test_fused_path_is_taken_and_matches_staged(scan):
    """The single-pass tcgen05 kernel against the staged kernels on the same inputs."""
    from frac_ssm_b200 import _cabi as C
    assert C.lib().fracssm_scan_fused_supported(6, 1000, 64, 128, 256, C.BF16, C.BF16) == 1
    u, c, kappa, rho, init = cuda(*O.scan_inputs(6, 1000, 64, 128, gen="model_like", seed=21))
    hf, ff = scan(u, c, kappa, rho, 256, init, True, final_state_dtype=torch.float32, path="fused", check=True)
    hs, fs = scan(u, c, kappa, rho, 256, init, True, final_state_dtype=torch.float32, path="staged")
    torch.testing.assert_close(hf.float(), hs.float(), **TOL_BF16)
    torch.testing.assert_close(ff, fs, **TOL_F32)
    with pytest.raises(Exception, match="not covered"):
        scan(u[:, :, :32].contiguous(), c, kappa, rho, 256, path="fused")


def test_fused_adversarial_decay(scan):
    """Modes pinned at the 1e-6 floor next to modes that never decay: the factorisation must stay
    finite and exact."""
    u, c, kappa, rho, _ = O.scan_inputs(2, 512, 64, 128, dtype=torch.bfloat16, gen="random", seed=5)
    rho[:, :, :64] = 1e-7
    rho[:, 40:400, 64:96] = 1.0
    rho[:, ::3, 96:] = 1e-6
    _check(scan, u, c, kappa, rho, 256, None, "fused")


def test_scan_inside_torch_compile_fullgraph(scan):
    """The scan is a registered custom op with a shape-only implementation, so a caller can compile
    a graph around it (the reference checks the same for its ops)."""
    u, c, kappa, rho, init = cuda(*O.scan_inputs(2, 512, 64, 128, gen="model_like", seed=17))

    def fn(u, c, kappa, rho, init):
        h, fin = scan(u * 1.0, c, kappa, rho, 256, init, True, final_state_dtype=torch.float32)
        return h.float() * 2.0, fin + 1.0

    eager = fn(u, c, kappa, rho, init)
    compiled = torch.compile(fn, fullgraph=True)(u, c, kappa, rho, init)
    torch.testing.assert_close(compiled[0], eager[0])
    torch.testing.assert_close(compiled[1], eager[1])
    with pytest.raises((NotImplementedError, RuntimeError)):
        ug = u.float().requires_grad_()          # forward only: gradients are refused
        scan(ug, c.float(), kappa.float(), rho, 256).sum().backward()


@pytest.mark.parametrize("B,L,ckdt", [(148, 256, torch.bfloat16), (16, 128, torch.bfloat16),
                                      (300, 257, torch.bfloat16), (96, 1024, torch.float32)])
def test_no_device_wait_runs_out_in_back_to_back_launches(B, L, ckdt):
    """Many launches queued without a host synchronisation, with other kernels in between (as inside
    a model): afterwards no launch may have recorded a device-side wait that ran out.  Guards the
    hand-over protocol of the single-pass kernel at CTA start-up, where a barrier once completed
    twice before a slow warp had looked at it."""
    import importlib
    FS = importlib.import_module("frac_ssm_b200.ops.b200.frac_scan")
    g = torch.Generator(device="cuda").manual_seed(B + L)
    u = (0.25 * torch.randn(B, L, 64, device="cuda", generator=g)).bfloat16()
    c = torch.softmax(torch.randn(B, L, 128, device="cuda", generator=g), -1).to(ckdt)
    k = (0.1 * torch.softmax(torch.randn(B, L, 128, device="cuda", generator=g), -1)).to(ckdt)
    rho = torch.rand(B, L, 128, device="cuda", generator=g).clamp(1e-6, 1 - 1e-6)
    filler = torch.randn(2048, 2048, device="cuda", dtype=torch.bfloat16)
    bad = torch.zeros((), device="cuda", dtype=torch.int64)    # a launch whose wait ran out writes NaN
    first = None
    for it in range(120):
        h = FS.frac_scan(u, c, k, rho, 256, None, False, path="fused")
        bad += torch.isnan(h).any()
        first = h if first is None else first
        if it % 3 == 0:
            filler = (filler @ filler) * 1e-3
    torch.cuda.synchronize()
    assert bad.item() == 0, f"{bad.item()} of 120 launches had a device-side wait run out"
    assert torch.equal(h, first)
