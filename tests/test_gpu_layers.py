"""Parity of the layer-level stages (parameter prep, skip-mix, gated RMSNorm, fused epilogue)."""

import os
import types

import pytest
import torch
import torch.nn.functional as F

from oracle import frac_oracle as O
from tests.helpers import TOL_BF16, TOL_F32, assert_ref_error, close

pytestmark = pytest.mark.gpu

CFG = dict(dt_min=1e-4, dt_max=1.0, alpha_min=0.2, alpha_max=0.95, lambda_min=0.25, lambda_max=4.0)


def _golden(golden_dir):
    return torch.load(os.path.join(golden_dir, "layer_small.pt"), weights_only=False)


def _mixer(g, device):
    """A stand-in for the reference's FracMixer holding just what the layer ops read."""
    m = g["meta"]
    mod = types.SimpleNamespace(num_heads=m["H"], head_dim=m["R"], num_modes=m["M"], read_temp=1.0)
    mod.dyn_proj = types.SimpleNamespace(weight=g["dyn_w"].to(device), bias=g["dyn_b"].to(device))
    mod.rw_proj = types.SimpleNamespace(weight=g["rw_w"].to(device))
    for k in ("dt_bias", "read_residual_logit", "write_residual_scale", "base_log_tau", "D"):
        setattr(mod, k, g[k].to(device))
    mod.config = types.SimpleNamespace(frac_dt_min=1e-4, frac_dt_max=1.0, frac_alpha_min=0.2,
                                       frac_alpha_max=0.95, frac_lambda_min=0.25, frac_lambda_max=4.0)
    return mod


@pytest.mark.parametrize("masked", [False, True])
def test_compute_params_on_golden(golden_dir, masked):
    from frac_ssm_b200.layers import frac_compute_scan_params
    g = _golden(golden_dir)
    mod = _mixer(g, "cuda")
    mask = g["mask"].cuda() if masked else None
    out = frac_compute_scan_params(mod, g["x_conv"].cuda(), g["x"].cuda(), mask)
    tag = "mask" if masked else "nomask"
    ref, pt = g[f"params_exact_{tag}"], g[f"params_work_{tag}"]
    for name, t in zip(("u", "c", "kappa", "rho"), out):
        close(t, ref[name], **TOL_F32)
        assert_ref_error(t, pt[name], ref[name], 1e-4)
    if masked:   # mask identity: kappa = 0 and rho = 1 where the mask is 0
        H = g["meta"]["H"]
        dead = (g["mask"] == 0)[:, None, :].expand(-1, H, -1).reshape(-1, g["mask"].shape[1])
        assert (out[2].cpu()[dead] == 0).all() and (out[3].cpu()[dead] == 1).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_compute_params_larger(dtype):
    from frac_ssm_b200.layers import compute_params_from_projections
    B, L, H, R, M = 2, 130, 6, 64, 128
    g = torch.Generator().manual_seed(2)
    dyn = torch.randn(B, L, 3 * H, generator=g).to(dtype)
    rw = torch.randn(B, L, 2 * H * M, generator=g).to(dtype)
    x = torch.randn(B, L, H * R, generator=g).to(dtype)
    dt_bias = torch.randn(H, generator=g)
    log_tau = torch.linspace(0.0, 11.09, M)
    args = (dt_bias, torch.tensor([-2.0]), torch.tensor([-1.1]), log_tau, H, R, M, 1.0,
            *CFG.values())
    out = compute_params_from_projections(dyn.cuda(), rw.cuda(), x.cuda(), None, dt_bias.cuda(), -2.0,
                                          -1.1, log_tau.cuda(), H, R, M, 1.0, *CFG.values())
    ref = O.compute_params(dyn.double(), rw.double(), x, None, *args, exact=True)
    pt = O.compute_params(dyn, rw, x, None, *args, exact=False)
    assert torch.equal(out[0].cpu(), pt[0].contiguous())
    for a, b, c_ in zip(out[1:], pt[1:], ref[1:]):
        close(a, c_, **TOL_F32)
        assert_ref_error(a, b, c_, 1e-4)


@pytest.mark.parametrize("M", [128, 16])
def test_compute_params_with_u_from_the_caller(M):
    """A caller that already holds the head-major u (the convolution writes it) gets the same
    coefficients, its own u back, and the kernel does not touch x_conv's copy."""
    from frac_ssm_b200.layers import compute_params_from_projections
    B, L, H, R = 2, 70, 4, 64
    g = torch.Generator().manual_seed(9)
    dyn = torch.randn(B, L, 3 * H, generator=g).bfloat16().cuda()
    rw = torch.randn(B, L, 2 * H * M, generator=g).bfloat16().cuda()
    x = torch.randn(B, L, H * R, generator=g).bfloat16().cuda()
    dt_bias = torch.randn(H, generator=g).cuda()
    log_tau = torch.linspace(0.0, 11.09, M).cuda()
    args = (dyn, rw, x, None, dt_bias, -2.0, -1.1, log_tau, H, R, M, 1.0, *CFG.values())
    u0, c0, k0, r0 = compute_params_from_projections(*args)
    mine = torch.full((B * H, L, R), 3.0, device="cuda", dtype=torch.bfloat16)
    u1, c1, k1, r1 = compute_params_from_projections(*args, u=mine)
    assert u1 is mine and torch.all(mine == 3.0)
    assert torch.equal(c0, c1) and torch.equal(k0, k1) and torch.equal(r0, r1)


@pytest.mark.parametrize("coeff", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("masked", [False, True])
def test_compute_params_128_modes_one_pass_kernel(coeff, masked):
    """bf16 projections with 128 modes take the vectorised one-pass kernel; L = 77 leaves a ragged
    group of tokens; the projections are strided views (as slices of a wider buffer)."""
    from frac_ssm_b200.layers import compute_params_from_projections
    B, L, H, R, M = 3, 77, 5, 64, 128
    g = torch.Generator().manual_seed(9)
    dyn = torch.randn(B, L, 3 * H, generator=g).bfloat16()
    rw_wide = torch.randn(B, L, 2 * H * M + 8, generator=g).bfloat16()
    rw = rw_wide[..., :2 * H * M]
    x = torch.randn(B, L, H * R, generator=g).bfloat16()
    mask = None
    if masked:
        mask = torch.ones(B, L)
        mask[0, :10] = 0
        mask[2, 50:] = 0
    dt_bias = torch.randn(H, generator=g)
    log_tau = torch.linspace(0.0, 11.09, M)
    args = (dt_bias, torch.tensor([-2.0]), torch.tensor([-1.1]), log_tau, H, R, M, 1.0, *CFG.values())
    out = compute_params_from_projections(dyn.cuda(), rw_wide.cuda()[..., :2 * H * M], x.cuda(),
                                          None if mask is None else mask.cuda(), dt_bias.cuda(), -2.0, -1.1,
                                          log_tau.cuda(), H, R, M, 1.0, *CFG.values(), coeff_dtype=coeff)
    ref = O.compute_params(dyn.double(), rw.double(), x, mask, *args, exact=True)
    assert out[1].dtype == coeff and out[2].dtype == coeff and out[3].dtype == torch.float32
    assert torch.equal(out[0].cpu(), x.view(B, L, H, R).permute(0, 2, 1, 3).reshape(B * H, L, R))
    tol = TOL_F32 if coeff == torch.float32 else dict(rtol=1e-2, atol=1e-4)
    close(out[1], ref[1], **tol)
    close(out[2], ref[2], **tol)
    close(out[3], ref[3], **TOL_F32)


def test_skip_mix_on_golden(golden_dir):
    from frac_ssm_b200.layers import frac_skip_mix
    g = _golden(golden_dir)
    mod = _mixer(g, "cuda")
    out = frac_skip_mix(mod, g["mixed_flat"].cuda(), g["x_conv"].cuda())
    close(out, g["mix_exact"], **TOL_F32)
    assert_ref_error(out, g["mix_work"], g["mix_exact"], 1e-4)
    out16 = frac_skip_mix(mod, g["mixed_flat"].cuda().bfloat16(), g["x_conv"].cuda().bfloat16())
    assert out16.dtype == torch.bfloat16
    close(out16, g["mix_exact"], rtol=3e-2, atol=3e-2)


def test_rmsnorm_gated_on_golden(golden_dir):
    from frac_ssm_b200.modules import MambaRMSNormGated, rmsnorm_gated_fwd
    g = _golden(golden_dir)
    x, gate, w = g["norm_x"].cuda(), g["norm_gate"].cuda(), g["norm_w"].cuda()
    y, rstd = rmsnorm_gated_fwd(x, w, gate, 1e-6)
    assert y.shape == x.shape and rstd.shape == x.shape[:-1] and y.dtype == x.dtype
    close(y, g["norm_exact"], **TOL_BF16)
    assert_ref_error(y, g["norm_work"], g["norm_exact"], 1e-3)
    y2, _ = rmsnorm_gated_fwd(x, w, None, 1e-6)
    close(y2, g["norm_work_nogate"], **TOL_BF16)
    mod = MambaRMSNormGated(48).cuda()
    close(mod(x.float(), gate.float()), O.rmsnorm_gated(x.float().cpu(), torch.ones(48), gate.float().cpu(),
                                                        exact=True), **TOL_F32)


@pytest.mark.parametrize("rows,D", [(1, 1536), (33, 1536), (7, 4096), (5, 100)])
def test_rmsnorm_gated_shapes(rows, D):
    from frac_ssm_b200.modules import rmsnorm_gated_fwd
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, D, generator=g).bfloat16()
    z = torch.randn(rows, D, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(D, generator=g)).bfloat16()
    y, rstd = rmsnorm_gated_fwd(x.cuda(), w.cuda(), z.cuda(), 1e-5)
    ref = O.rmsnorm_gated(x, w, z, 1e-5, exact=True)
    close(y, ref, **TOL_BF16)
    v = (x.double() * F.silu(z.double()))
    close(rstd, torch.rsqrt(v.pow(2).mean(-1) + 1e-5), **TOL_F32)


@pytest.mark.parametrize("rows,D,gated", [(1, 768, False), (37, 768, True), (130, 1536, True), (5, 2048, False),
                                          (9, 8, True), (3, 2056, True)])
def test_rmsnorm_bf16_row_in_registers(rows, D, gated):
    """Widths up to 2048 in bf16 take the warp-per-row kernel (2056 falls back to the general one);
    x and the gate are strided row views."""
    from frac_ssm_b200.modules import rmsnorm_gated_fwd
    g = torch.Generator().manual_seed(rows + D)
    both = torch.randn(rows, 2 * D, generator=g).bfloat16()
    x, z = both[:, :D], both[:, D:]
    w = (1 + 0.1 * torch.randn(D, generator=g)).bfloat16()
    bc = both.cuda()
    y, rstd = rmsnorm_gated_fwd(bc[:, :D], w.cuda(), bc[:, D:] if gated else None, 1e-6)
    ref = O.rmsnorm_gated(x, w, z if gated else None, 1e-6, exact=True)
    close(y, ref, **TOL_BF16)
    v = x.double() * F.silu(z.double()) if gated else x.double()
    close(rstd, torch.rsqrt(v.pow(2).mean(-1) + 1e-6), **TOL_F32)


def test_scan_epilogue_matches_unfused_pair():
    from frac_ssm_b200.layers import scan_epilogue
    B, L, H, R = 2, 50, 24, 64
    g = torch.Generator().manual_seed(3)
    h = torch.randn(B * H, L, R, generator=g).bfloat16()
    x = torch.randn(B, L, H * R, generator=g).bfloat16()
    z = torch.randn(B, L, H * R, generator=g).bfloat16()
    D = torch.randn(H, R, generator=g)
    w = (1 + 0.1 * torch.randn(H * R, generator=g)).bfloat16()
    y = scan_epilogue(h.cuda(), x.cuda(), z.cuda(), D.cuda(), w.cuda(), H, R, 1e-6, gate_bias=0.5)
    mixed = O.skip_mix(h, x, D, H, R, exact=True)
    ref = O.rmsnorm_gated(mixed, w, z.double() + 0.5, 1e-6, exact=True)
    close(y, ref, **TOL_BF16)


@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,L,H,R", [(1, 1, 4, 64), (3, 7, 3, 40), (2, 21, 32, 64), (1, 130, 24, 64), (2, 9, 40, 64)])
def test_scan_epilogue_row_widths(B, L, H, R, wdtype):
    """Row widths on either side of each register-resident variant (256, 120, 2048, 1536 columns) and
    one beyond them (2560), row counts that do not fill the last block, both weight types."""
    from frac_ssm_b200.layers import scan_epilogue
    g = torch.Generator().manual_seed(17)
    h = torch.randn(B * H, L, R, generator=g).bfloat16()
    x = torch.randn(B, L, H * R, generator=g).bfloat16()
    z = torch.randn(B, L, H * R, generator=g).bfloat16()
    D = torch.randn(H, R, generator=g)
    w = (1 + 0.1 * torch.randn(H * R, generator=g)).to(wdtype)
    y = scan_epilogue(h.cuda(), x.cuda(), z.cuda(), D.cuda(), w.cuda(), H, R, 1e-6, gate_bias=-0.25)
    ref = O.rmsnorm_gated(O.skip_mix(h, x, D, H, R, exact=True), w, z.double() - 0.25, 1e-6, exact=True)
    close(y, ref, **TOL_BF16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shards", [2, 3, 8])
def test_head_sharded_epilogue_two_passes(dtype, shards):
    """Partial sums of squares per head shard, added, then applied: same result as the one-pass
    epilogue over all heads (the shards are emulated one after another on this GPU)."""
    from frac_ssm_b200.layers import scan_epilogue, scan_epilogue_apply, scan_epilogue_sumsq
    from frac_ssm_b200.parallel import shard_heads
    B, L, H, R = 2, 37, 24, 64
    g = torch.Generator().manual_seed(5)
    h = torch.randn(B * H, L, R, generator=g).to(dtype).cuda()
    x = torch.randn(B, L, H * R, generator=g).to(dtype).cuda()
    z = torch.randn(B, L, H * R, generator=g).to(dtype).cuda()
    D = torch.randn(H, R, generator=g).cuda()
    w = (1 + 0.1 * torch.randn(H * R, generator=g)).to(dtype).cuda()
    y_full = scan_epilogue(h, x, z, D, w, H, R, 1e-6, gate_bias=0.25)
    parts, total = [], torch.zeros(B, L, device="cuda")
    for r in range(shards):
        hs = shard_heads(H, r, shards)
        n, cols = hs.stop - hs.start, slice(hs.start * R, hs.stop * R)
        h_loc = h.view(B, H, L, R)[:, hs].reshape(B * n, L, R)
        args = (h_loc, x[..., cols], z[..., cols], D[hs])      # column slices stay strided views
        parts.append((args, w[cols], n, cols))
        total += scan_epilogue_sumsq(*args, n, R, gate_bias=0.25)
    ref = O.rmsnorm_gated(O.skip_mix(h.cpu(), x.cpu(), D.cpu(), H, R, exact=True), w.cpu(),
                          z.cpu().double() + 0.25, 1e-6, exact=True)
    for args, w_loc, n, cols in parts:
        y = scan_epilogue_apply(*args, w_loc, n, R, total, H * R, 1e-6, gate_bias=0.25)
        close(y, ref[..., cols], **(TOL_BF16 if dtype == torch.bfloat16 else TOL_F32))
        close(y, y_full[..., cols].float().cpu(), rtol=1e-2 if dtype == torch.bfloat16 else 1e-5,
              atol=1e-2 if dtype == torch.bfloat16 else 1e-5)


def test_mixer_path_composition_matches_oracle():
    """The whole layer path as FracMixer.forward strings it together (prep -> scan -> skip-mix ->
    gated norm) on the CUDA ops, against the same composition on the CPU oracle."""
    from frac_ssm_b200.layers import compute_params_from_projections, frac_skip_mix, scan_epilogue
    from frac_ssm_b200.modules import rmsnorm_gated_fwd
    from frac_ssm_b200.ops import frac_scan
    B, L, H, R, M, T = 2, 600, 4, 64, 128, 256
    g = torch.Generator().manual_seed(9)
    dyn = torch.randn(B, L, 3 * H, generator=g).bfloat16()
    rw = torch.randn(B, L, 2 * H * M, generator=g).bfloat16()
    x_conv = torch.randn(B, L, H * R, generator=g).bfloat16()
    gate = torch.randn(B, L, H * R, generator=g).bfloat16()
    dt_bias = torch.randn(H, generator=g) - 2.0
    log_tau = torch.linspace(0.0, 11.09, M)
    D = torch.randn(H, R, generator=g)
    w = (1 + 0.1 * torch.randn(H * R, generator=g)).bfloat16()
    pargs = (H, R, M, 1.0, *CFG.values())

    u, c, kappa, rho = compute_params_from_projections(
        dyn.cuda(), rw.cuda(), x_conv.cuda(), None, dt_bias.cuda(), -2.0, -1.1, log_tau.cuda(), *pargs)
    h = frac_scan(u, c, kappa, rho, T)                       # fp32 c / kappa with bf16 u: the model's case
    mod = types.SimpleNamespace(D=D.cuda(), num_heads=H, head_dim=R)
    mixed = frac_skip_mix(mod, h, x_conv.cuda())
    y, _ = rmsnorm_gated_fwd(mixed, w.cuda(), gate.cuda(), 1e-6)
    y_fused = scan_epilogue(h, x_conv.cuda(), gate.cuda(), D.cuda(), w.cuda(), H, R, 1e-6)

    uo, co, ko, ro = O.compute_params(dyn.double(), rw.double(), x_conv, None, dt_bias, torch.tensor([-2.0]),
                                      torch.tensor([-1.1]), log_tau, *pargs, exact=True)
    ho = O.frac_scan_slabs(uo.float(), co.float(), ko.float(), ro.float(), T, None, False, exact=True, slab=2)
    mo = O.skip_mix(ho, x_conv, D, H, R, exact=True)
    yo = O.rmsnorm_gated(mo, w, gate, 1e-6, exact=True)
    close(h, ho, **TOL_BF16)
    close(y, yo, rtol=3e-2, atol=3e-2)       # two bf16 roundings (h, mixed) before the norm
    close(y_fused, yo, **TOL_BF16)


@pytest.mark.parametrize("B,H,L,with_init,ckdt", [(2, 3, 700, True, torch.bfloat16), (1, 4, 129, False, torch.float32),
                                                   (3, 2, 1024, False, torch.bfloat16)])
def test_fused_layer_path_matches_oracle(B, H, L, with_init, ckdt):
    """Scan with the skip-mix and the gate fused into its output stage, then the norm pass: against
    rmsnorm_gated(skip_mix(frac_scan(...))) of the oracle, on ragged L, with and without an initial
    state; and the plain frac_scan still returns h as before."""
    from frac_ssm_b200.layers import scan_layer
    from frac_ssm_b200.ops.b200 import frac_scan
    R, M, T = 64, 128, 256
    u, c, kappa, rho, init = O.scan_inputs(B * H, L, R, M, dtype=torch.bfloat16, gen="model_like", seed=41)
    init = init if with_init else None
    g = torch.Generator().manual_seed(42)
    gate = torch.randn(B, L, H * R, generator=g).bfloat16()
    D = torch.randn(H, R, generator=g)
    w = (torch.rand(H * R, generator=g) + 0.5).bfloat16()
    x_conv = u.view(B, H, L, R).permute(0, 2, 1, 3).reshape(B, L, H * R)
    h_ref, f_ref = O.frac_scan_slabs(u.float(), c.float(), kappa.float(), rho, T, init, True, exact=True, slab=2)
    y_ref = O.rmsnorm_gated(O.skip_mix(h_ref, x_conv, D, H, R, exact=True), w, gate.float() + 0.25, 1e-6, exact=True)
    cg, kg = c.to(ckdt).cuda(), kappa.to(ckdt).cuda()
    y, fin = scan_layer(u.cuda(), cg, kg, rho.cuda(), gate.cuda(), D.cuda(), w.cuda(), H, 1e-6, 0.25,
                        None if init is None else init.cuda(), True)
    close(y, y_ref, rtol=3e-2, atol=3e-2)      # two bf16 roundings (the gated values, then y) around the norm
    close(fin, f_ref, **TOL_F32)
    h = frac_scan(u.cuda(), cg, kg, rho.cuda(), T, None if init is None else init.cuda(), False)
    close(h, h_ref, **TOL_BF16)


@pytest.mark.parametrize("shards", [2, 4])
def test_fused_layer_path_head_sharded_emulation(shards):
    """The head-sharded form on one GPU: every shard's scan + gate pass, the shards' row sums added by hand
    (what the all-reduce does), every shard normalised with the total: equals the unsharded fused layer."""
    from frac_ssm_b200.layers import scan_layer, scan_layer_gated, scan_layer_norm, scan_layer_sumsq
    B, H, L, R, M = 2, 8, 300, 64, 128
    u, c, kappa, rho, _ = (t.cuda() for t in O.scan_inputs(B * H, L, R, M, dtype=torch.bfloat16, gen="random", seed=43))
    g = torch.Generator().manual_seed(44)
    gate = torch.randn(B, L, H * R, generator=g).bfloat16().cuda()
    D = torch.randn(H, R, generator=g).cuda()
    w = (torch.rand(H * R, generator=g) + 0.5).bfloat16().cuda()
    y_full = scan_layer(u, c, kappa, rho, gate, D, w, H, 1e-6, 0.0)
    hl = H // shards
    parts = []
    for s in range(shards):
        rows = lambda t: t.view(B, H, L, -1)[:, s * hl:(s + 1) * hl].reshape(B * hl, L, -1).contiguous()
        cols = slice(s * hl * R, (s + 1) * hl * R)
        gated, ss, _ = scan_layer_gated(rows(u), rows(c), rows(kappa), rows(rho), gate[..., cols].contiguous(),
                                        D[s * hl:(s + 1) * hl], hl, 0.0)
        parts.append((gated, ss, cols))
    total = sum(scan_layer_sumsq(ss) for _, ss, _ in parts)
    for gated, ss, cols in parts:
        y = scan_layer_norm(gated, ss, w[cols], R, 1e-6, sumsq=total, norm_width=H * R)
        torch.testing.assert_close(y.float(), y_full[..., cols].float(), rtol=1e-2, atol=1e-3)


def test_frac_compute_scan_params_does_not_synchronise():
    """The drop-in entry point takes the two scalar gate parameters as device tensors, like the
    reference (its layers/compute_params.py:199-202): no host read, so no synchronisation."""
    from frac_ssm_b200.layers import frac_compute_scan_params
    H, R, M, hidden = 2, 64, 128, 96
    torch.manual_seed(5)
    cfg = types.SimpleNamespace(frac_dt_min=1e-4, frac_dt_max=1.0, frac_alpha_min=0.2, frac_alpha_max=0.95,
                                frac_lambda_min=0.25, frac_lambda_max=4.0)
    mixer = types.SimpleNamespace(
        dyn_proj=torch.nn.Linear(hidden, 3 * H).cuda().bfloat16(), rw_proj=torch.nn.Linear(H * R, 2 * H * M, bias=False).cuda().bfloat16(),
        dt_bias=torch.randn(H, device="cuda") - 2.0, read_residual_logit=torch.nn.Parameter(torch.tensor([-2.0], device="cuda")),
        write_residual_scale=torch.nn.Parameter(torch.tensor([-1.1], device="cuda")),
        base_log_tau=torch.linspace(0.0, 11.09, M, device="cuda"), num_heads=H, head_dim=R, num_modes=M, read_temp=1.0, config=cfg)
    x = torch.randn(2, 40, hidden, device="cuda").bfloat16()
    x_conv = torch.randn(2, 40, H * R, device="cuda").bfloat16()
    with torch.no_grad():
        frac_compute_scan_params(mixer, x_conv, x)            # warm-up: library load, cuBLAS handles
        torch.cuda.synchronize()
        torch.cuda.set_sync_debug_mode("error")
        try:
            u, c, kappa, rho = frac_compute_scan_params(mixer, x_conv, x)
        finally:
            torch.cuda.set_sync_debug_mode("default")
    assert u.shape == (2 * H, 40, R) and rho.dtype == torch.float32 and torch.isfinite(c).all()
