"""Generate the golden fixtures in this folder from the reference implementation.

Run where the reference checkout is available (it is not needed to run the tests):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/frac-ssm-kernels

It imports the reference's pure-PyTorch functions (`frac_ssm.ops.refs.*`,
`frac_ssm.layers.refs.*`, `frac_ssm.modules.rmsnorm_gated.rmsnorm_gated_ref`), runs
them on small seeded CPU inputs, and stores inputs and outputs with `torch.save`.
The inputs come from the generators in `oracle/frac_oracle.py` (CPU generators) and are
stored too, so the fixtures do not depend on the random number stream.
"""

from __future__ import annotations

import argparse
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def scan_case(refs, name, B, L, R, M, T, dtype, gen, seed, with_init):
    from oracle import frac_oracle as O

    u, c, kappa, rho, init = O.scan_inputs(B, L, R, M, dtype=dtype, gen=gen, seed=seed)
    init = init if with_init else None
    out = {"meta": dict(B=B, L=L, R=R, M=M, T=T, gen=gen, seed=seed),
           "u": u, "c": c, "kappa": kappa, "rho": rho, "initial_state": init}
    for tag, up in (("work", False), ("exact", True)):
        if up:
            uu, cc, kk = u.float(), c.float(), kappa.float()
        else:
            uu, cc, kk = u, c, kappa
        log_rho = (torch.log(rho.double().clamp(min=1e-6)).float() if up
                   else torch.log(rho.clamp(min=1e-6)))
        lcr, cd = refs["cumsum"](log_rho, T, upcast=up)
        st = refs["state"](uu, kk, lcr, T, state_fp32=up or uu.dtype != torch.bfloat16, upcast=up)
        acc, fin = refs["passing"](st, cd, init, upcast=up)
        W = refs["w"](cc, kk, lcr, T, upcast=up)
        h = refs["readout"](uu, cc, acc, W, lcr, T, upcast=up)
        h2, fin2 = refs["scan"](uu, cc, kk, rho, T, init, True, upcast=up)
        assert torch.equal(h, h2) and torch.equal(fin, fin2)
        out[tag] = {"lcr": lcr, "chunk_decay": cd, "states": st, "states_acc": acc,
                    "final_state": fin, "W": W, "h": h}
    torch.save(out, os.path.join(HERE, name + ".pt"))
    print("wrote", name)


def config0_case(refs):
    """BASELINE config 0 (batch 1, L 1024, H 8, R 64, M 64, T 64, fp32, seed 0):
    outputs are stored subsampled to keep the fixture small."""
    from oracle import frac_oracle as O

    d = O.layer_inputs(1, 1024, 8, 64, 64, G=1, seed=0, dtype=torch.float32)
    u, c, kappa, rho = d["u"], d["c"], d["kappa"], d["rho"]
    out = {"meta": dict(batch=1, L=1024, H=8, R=64, M=64, T=64, seed=0)}
    for tag, up in (("work", False), ("exact", True)):
        h, fin = refs["scan"](u, c, kappa, rho, 64, None, True, upcast=up)
        out[tag] = {"h_sub": h[:, ::37, ::5].contiguous(), "final_sub": fin[:, ::3, ::7].contiguous(),
                    "h_sum": h.double().sum(), "h_abs_sum": h.double().abs().sum()}
    # input fingerprints so a drifting random stream is detected, not silently compared
    out["fingerprint"] = {k: d[k].double().sum() for k in ("u", "c", "kappa", "rho")}
    torch.save(out, os.path.join(HERE, "config0_subsample.pt"))
    print("wrote config0_subsample")


def layer_case(refs):
    import torch.nn as nn

    torch.manual_seed(5)
    B, L, H, R, M = 2, 37, 3, 8, 16
    inner = H * R
    model = types.SimpleNamespace()
    model.num_heads, model.head_dim, model.num_modes, model.inner_dim = H, R, M, inner
    model.read_temp = 1.0
    model.dyn_proj = nn.Linear(inner, 3 * H, bias=True)
    model.rw_proj = nn.Linear(inner, 2 * H * M, bias=False)
    model.dt_bias = torch.randn(H) * 0.5
    model.read_residual_logit = torch.tensor([-2.0])
    model.write_residual_scale = torch.tensor([-1.0986])
    model.base_log_tau = torch.linspace(0.0, 11.09, M)
    model.D = torch.randn(H, R)
    model.config = types.SimpleNamespace(
        frac_dt_min=1e-4, frac_dt_max=1.0, frac_alpha_min=0.2, frac_alpha_max=0.95,
        frac_lambda_min=0.25, frac_lambda_max=4.0)
    x = torch.randn(B, L, inner)
    x_conv = torch.randn(B, L, inner)
    mask = (torch.rand(B, L) > 0.2).float()
    out = {"meta": dict(B=B, L=L, H=H, R=R, M=M), "x": x, "x_conv": x_conv, "mask": mask,
           "dyn_w": model.dyn_proj.weight.detach(), "dyn_b": model.dyn_proj.bias.detach(),
           "rw_w": model.rw_proj.weight.detach(), "dt_bias": model.dt_bias,
           "read_residual_logit": model.read_residual_logit,
           "write_residual_scale": model.write_residual_scale,
           "base_log_tau": model.base_log_tau, "D": model.D}
    with torch.no_grad():
        for tag, up in (("work", False), ("exact", True)):
            for mtag, mk in (("nomask", None), ("mask", mask)):
                uf, cf, kf, rf = refs["params"](model, x_conv, x, mk, upcast=up)
                out[f"params_{tag}_{mtag}"] = {"u": uf.contiguous(), "c": cf.contiguous(),
                                               "kappa": kf.contiguous(), "rho": rf.contiguous()}
            mixed_flat = torch.randn(B * H, L, R)
            out["mixed_flat"] = mixed_flat if "mixed_flat" not in out else out["mixed_flat"]
            out[f"mix_{tag}"] = refs["mix"](model, out["mixed_flat"], x_conv, None, upcast=up)
        xs = torch.randn(5, 11, 48).to(torch.bfloat16)
        gate = torch.randn(5, 11, 48).to(torch.bfloat16)
        w = (1.0 + 0.1 * torch.randn(48)).to(torch.bfloat16)
        out["norm_x"], out["norm_gate"], out["norm_w"] = xs, gate, w
        out["norm_work"] = refs["norm"](xs, w, gate, 1e-6, upcast=False)
        out["norm_exact"] = refs["norm"](xs, w, gate, 1e-6, upcast=True)
        out["norm_work_nogate"] = refs["norm"](xs, w, None, 1e-6, upcast=False)
    torch.save(out, os.path.join(HERE, "layer_small.pt"))
    print("wrote layer_small")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    sys.path.insert(0, ROOT)
    sys.path.insert(0, args.reference)

    from frac_ssm.ops.refs.chunk_cumsum import chunk_cumsum_ref
    from frac_ssm.ops.refs.chunk_state import chunk_state_ref
    from frac_ssm.ops.refs.state_passing import state_passing_ref
    from frac_ssm.ops.refs.chunk_w import chunk_w_ref
    from frac_ssm.ops.refs.chunk_readout import chunk_readout_ref
    from frac_ssm.ops.refs.frac_scan import frac_scan_ref
    from frac_ssm.layers.refs import frac_compute_scan_params_ref, frac_skip_mix_ref
    from frac_ssm.modules.rmsnorm_gated import rmsnorm_gated_ref

    refs = {"cumsum": chunk_cumsum_ref, "state": chunk_state_ref, "passing": state_passing_ref,
            "w": chunk_w_ref, "readout": chunk_readout_ref, "scan": frac_scan_ref,
            "params": frac_compute_scan_params_ref, "mix": frac_skip_mix_ref,
            "norm": rmsnorm_gated_ref}
    torch.set_num_threads(1)
    scan_case(refs, "scan_f32_ragged", 3, 70, 8, 8, 16, torch.float32, "model_like", 0, True)
    scan_case(refs, "scan_f32_random", 2, 64, 16, 8, 32, torch.float32, "random", 3, False)
    scan_case(refs, "scan_bf16_init", 2, 96, 16, 16, 32, torch.bfloat16, "model_like", 1, True)
    scan_case(refs, "scan_bf16_ragged", 2, 45, 8, 16, 16, torch.bfloat16, "random", 2, False)
    config0_case(refs)
    layer_case(refs)


if __name__ == "__main__":
    main()
