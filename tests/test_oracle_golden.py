"""The CPU oracle against outputs of the reference implementation (tests/golden/*.pt)."""

import os

import pytest
import torch

from oracle import frac_oracle as O

SCAN_CASES = ["scan_f32_ragged", "scan_f32_random", "scan_bf16_init", "scan_bf16_ragged"]


def _load(golden_dir, name):
    return torch.load(os.path.join(golden_dir, name + ".pt"), weights_only=False)


def _close(a, b, tol=1e-6):
    assert a.shape == b.shape and a.dtype == b.dtype
    torch.testing.assert_close(a.double(), b.double(), rtol=tol, atol=tol)


@pytest.mark.parametrize("name", SCAN_CASES)
@pytest.mark.parametrize("mode", ["work", "exact"])
def test_scan_stages_match_reference(golden_dir, name, mode):
    g = _load(golden_dir, name)
    exact = mode == "exact"
    T = g["meta"]["T"]
    u, c, kappa, rho, init = g["u"], g["c"], g["kappa"], g["rho"], g["initial_state"]
    if exact:
        u, c, kappa = u.float(), c.float(), kappa.float()
    ref = g[mode]
    lcr, cd = O.chunk_cumsum(O.log_decay(rho, exact), T, exact)
    _close(lcr, ref["lcr"])
    _close(cd, ref["chunk_decay"])
    st = O.chunk_state(u, kappa, ref["lcr"], T, state_fp32=exact or u.dtype != torch.bfloat16,
                       exact=exact)
    # bf16 working precision: one bf16 ulp of slack for reduction-order differences
    tol = 1e-6 if st.dtype == torch.float32 else 1e-2
    _close(st, ref["states"], tol)
    acc, fin = O.state_passing(ref["states"], ref["chunk_decay"], init, exact=exact)
    _close(acc, ref["states_acc"], tol)
    _close(fin, ref["final_state"], tol)
    W = O.chunk_w(c, kappa, ref["lcr"], T, exact)
    _close(W, ref["W"])
    h = O.chunk_readout(u, c, ref["states_acc"], ref["W"], ref["lcr"], T, exact)
    _close(h, ref["h"], tol)
    h2, fin2 = O.frac_scan(u, c, kappa, rho, T, init, True, exact)
    _close(h2, ref["h"], tol)
    _close(fin2, ref["final_state"], tol)
    h3, fin3 = O.frac_scan_slabs(u, c, kappa, rho, T, init, True, exact, slab=1)
    _close(h3, ref["h"], tol)


@pytest.mark.parametrize("name", SCAN_CASES)
def test_exact_mode_equals_token_recurrence(golden_dir, name):
    g = _load(golden_dir, name)
    u, c, kappa, rho, init = g["u"], g["c"], g["kappa"], g["rho"], g["initial_state"]
    h, fin = O.token_recurrence(u, c, kappa, rho, init)
    torch.testing.assert_close(g["exact"]["h"].double(), h, rtol=2e-4, atol=2e-4)
    torch.testing.assert_close(g["exact"]["final_state"].double(), fin, rtol=2e-4, atol=2e-4)


def test_config0_matches_reference(golden_dir):
    g = _load(golden_dir, "config0_subsample")
    d = O.layer_inputs(1, 1024, 8, 64, 64, G=1, seed=0, dtype=torch.float32)
    for k, v in g["fingerprint"].items():
        torch.testing.assert_close(d[k].double().sum(), v, rtol=1e-9, atol=1e-9)
    for mode in ("work", "exact"):
        h, fin = O.frac_scan(d["u"], d["c"], d["kappa"], d["rho"], 64, None, True, mode == "exact")
        _close(h[:, ::37, ::5].contiguous(), g[mode]["h_sub"], 2e-6)
        _close(fin[:, ::3, ::7].contiguous(), g[mode]["final_sub"], 2e-6)
        torch.testing.assert_close(h.double().sum(), g[mode]["h_sum"], rtol=1e-6, atol=1e-4)


def test_layer_stages_match_reference(golden_dir):
    g = _load(golden_dir, "layer_small")
    m = g["meta"]
    H, R, M = m["H"], m["R"], m["M"]
    for mode in ("work", "exact"):
        exact = mode == "exact"
        if exact:
            dyn = torch.nn.functional.linear(g["x"].double(), g["dyn_w"].double(), g["dyn_b"].double())
            rw = torch.nn.functional.linear(g["x_conv"].double(), g["rw_w"].double())
        else:
            dyn = torch.nn.functional.linear(g["x"], g["dyn_w"], g["dyn_b"])
            rw = torch.nn.functional.linear(g["x_conv"], g["rw_w"])
        for mtag, mask in (("nomask", None), ("mask", g["mask"])):
            got = O.compute_params(dyn, rw, g["x_conv"], mask, g["dt_bias"],
                                   g["read_residual_logit"], g["write_residual_scale"],
                                   g["base_log_tau"], H, R, M, 1.0, 1e-4, 1.0, 0.2, 0.95, 0.25, 4.0,
                                   exact=exact)
            ref = g[f"params_{mode}_{mtag}"]
            for name, t in zip(("u", "c", "kappa", "rho"), got):
                _close(t.contiguous(), ref[name], 1e-6)
        mix = O.skip_mix(g["mixed_flat"], g["x_conv"], g["D"], H, R, None, exact=exact)
        _close(mix, g[f"mix_{mode}"], 1e-6)
    _close(O.rmsnorm_gated(g["norm_x"], g["norm_w"], g["norm_gate"], 1e-6, False), g["norm_work"], 1e-2)
    _close(O.rmsnorm_gated(g["norm_x"], g["norm_w"], g["norm_gate"], 1e-6, True), g["norm_exact"], 1e-9)
    _close(O.rmsnorm_gated(g["norm_x"], g["norm_w"], None, 1e-6, False), g["norm_work_nogate"], 1e-2)


def test_cumsum_reconstructs_full_sequence_sum():
    # per-chunk sums plus the totals of the chunks before them give the full running sum
    lr = O.model_like_log_rho(2, 100, 8, seed=4)
    lcr, cd = O.chunk_cumsum(lr, 16)
    full = lr.double().cumsum(1)
    offs = torch.cat([torch.zeros(2, 1, 8, dtype=torch.float64), cd.double().cumsum(1)[:, :-1]], 1)
    rebuilt = lcr.double() + offs.repeat_interleave(16, dim=1)[:, :100]
    torch.testing.assert_close(rebuilt, full, rtol=1e-5, atol=1e-4)
