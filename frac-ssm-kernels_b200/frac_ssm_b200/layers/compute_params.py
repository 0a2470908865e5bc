"""Scan-parameter prep on the B200 CUDA extension.

Interface of `frac_ssm/layers/compute_params.py:583-596`: the two projections stay library
GEMMs (`F.linear`), everything after them is one kernel.  Forward only.
"""

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .. import _cabi as C
from ..ops.b200.stages import _op


def compute_params_from_projections(dyn, rw, x_conv, attention_mask, dt_bias, read_residual_logit,
                                    write_residual_scale, base_log_tau, num_heads, head_dim,
                                    num_modes, read_temp, dt_min, dt_max, alpha_min, alpha_max,
                                    lambda_min, lambda_max, coeff_dtype=torch.float32, u=None):
    """Elementwise part: dyn [B,L,3H], rw [B,L,2HM], x_conv [B,L,HR] ->
    (u [BH,L,R] in x_conv.dtype, c, kappa [BH,L,M] in `coeff_dtype`, rho [BH,L,M] float32),
    head-major.  The reference emits float32 coefficients; bfloat16 halves what the scan reads.
    `read_residual_logit` / `write_residual_scale` are the two scalar parameters as tensors (they
    stay on the device: nothing here synchronises) or, for convenience, Python numbers.
    `u`: the head-major copy of x_conv when the caller already has it (the convolution can write
    it): it is returned as it is and the kernel neither reads x_conv nor writes u."""
    assert dyn.dim() == 3 and rw.dim() == 3 and x_conv.dim() == 3, "dyn, rw and x_conv must be 3D"
    assert dyn.is_cuda and rw.is_cuda and x_conv.is_cuda, "inputs must be on CUDA"
    B, L, _ = x_conv.shape
    H, R, M = num_heads, head_dim, num_modes
    assert dyn.shape == (B, L, 3 * H), "dyn shape must be (B, L, 3*H)"
    assert rw.shape == (B, L, 2 * H * M), "rw shape must be (B, L, 2*H*M)"
    assert x_conv.shape == (B, L, H * R), "x_conv shape must be (B, L, H*R)"
    dev = x_conv.device
    mask = None
    if attention_mask is not None:
        assert attention_mask.shape == (B, L), "attention_mask shape must be (B, L)"
        mask = attention_mask.to(device=dev, dtype=torch.float32)

    def scalar(v):
        if torch.is_tensor(v):
            return v.detach().to(device=dev, dtype=torch.float32).reshape(-1)[:1].contiguous()
        return torch.full((1,), float(v), device=dev, dtype=torch.float32)

    args = (dyn, rw, x_conv, mask, dt_bias.detach().to(device=dev, dtype=torch.float32).contiguous(),
            scalar(read_residual_logit), scalar(write_residual_scale),
            base_log_tau.detach().to(device=dev, dtype=torch.float32).contiguous(), H, R, M, float(read_temp),
            float(dt_min), float(dt_max), float(alpha_min), float(alpha_max), float(lambda_min), float(lambda_max),
            coeff_dtype)
    if u is not None:
        assert u.shape == (B * H, L, R) and u.dtype == x_conv.dtype and u.is_cuda, "u must be (B*H, L, R) like x_conv"
        c, kappa, rho = _compute_coeffs_op(*args)
        return u, c, kappa, rho
    u, c, kappa, rho = _compute_params_op(*args)
    return u, c, kappa, rho


def _launch_params(dyn, rw, x_conv, mask, dtb, rlog, wlog, ltau, H, R, M, read_temp, dt_min, dt_max, alpha_min,
                   alpha_max, lambda_min, lambda_max, coeff_dtype, want_u):
    B, L, _ = x_conv.shape
    dev = x_conv.device
    dyn, rw, x_conv = C.rows(dyn), C.rows(rw), C.rows(x_conv)
    u = torch.empty(B * H, L, R, device=dev, dtype=x_conv.dtype) if want_u else None
    c = torch.empty(B * H, L, M, device=dev, dtype=coeff_dtype)
    kappa = torch.empty_like(c)
    rho = torch.empty(B * H, L, M, device=dev, dtype=torch.float32)
    if B == 0 or L == 0:
        return u, c, kappa, rho
    with C.trace("frac_compute_scan_params"), torch.cuda.device(dev):
        C.check(C.lib().fracssm_compute_params(
            C.ptr(dyn), C.dt(dyn), dyn.stride(0), dyn.stride(1), C.ptr(rw), C.dt(rw), rw.stride(0),
            rw.stride(1), C.ptr(x_conv), C.dt(x_conv), x_conv.stride(0), x_conv.stride(1),
            C.ptr(mask), 0 if mask is None else mask.stride(0), 0 if mask is None else mask.stride(1),
            C.ptr(dtb), C.ptr(ltau), C.ptr(rlog), C.ptr(wlog),
            float(read_temp), float(dt_min), float(dt_max), float(alpha_min), float(alpha_max),
            float(lambda_min), float(lambda_max), C.ptr(u), C.ptr(c), C.ptr(kappa), C.dt(c), C.ptr(rho),
            B, L, H, R, M, C.stream_of(x_conv)), "compute_params")
    return u, c, kappa, rho


# torch custom ops with shape-only implementations (torch.compile(fullgraph=True)); forward only
@_op("compute_params")
def _compute_params_op(dyn: torch.Tensor, rw: torch.Tensor, x_conv: torch.Tensor, mask: Optional[torch.Tensor],
                       dtb: torch.Tensor, rlog: torch.Tensor, wlog: torch.Tensor, ltau: torch.Tensor, H: int, R: int,
                       M: int, read_temp: float, dt_min: float, dt_max: float, alpha_min: float, alpha_max: float,
                       lambda_min: float, lambda_max: float, coeff_dtype: torch.dtype
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return _launch_params(dyn, rw, x_conv, mask, dtb, rlog, wlog, ltau, H, R, M, read_temp, dt_min, dt_max,
                          alpha_min, alpha_max, lambda_min, lambda_max, coeff_dtype, True)


@_compute_params_op.register_fake
def _(dyn, rw, x_conv, mask, dtb, rlog, wlog, ltau, H, R, M, read_temp, dt_min, dt_max, alpha_min, alpha_max,
      lambda_min, lambda_max, coeff_dtype):
    B, L, _ = x_conv.shape
    dev = x_conv.device
    c = torch.empty(B * H, L, M, device=dev, dtype=coeff_dtype)
    return (torch.empty(B * H, L, R, device=dev, dtype=x_conv.dtype), c, torch.empty_like(c),
            torch.empty(B * H, L, M, device=dev, dtype=torch.float32))


# the same without the head-major copy of x_conv (the caller has u already)
@_op("compute_coeffs")
def _compute_coeffs_op(dyn: torch.Tensor, rw: torch.Tensor, x_conv: torch.Tensor, mask: Optional[torch.Tensor],
                       dtb: torch.Tensor, rlog: torch.Tensor, wlog: torch.Tensor, ltau: torch.Tensor, H: int, R: int,
                       M: int, read_temp: float, dt_min: float, dt_max: float, alpha_min: float, alpha_max: float,
                       lambda_min: float, lambda_max: float, coeff_dtype: torch.dtype
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _launch_params(dyn, rw, x_conv, mask, dtb, rlog, wlog, ltau, H, R, M, read_temp, dt_min, dt_max,
                          alpha_min, alpha_max, lambda_min, lambda_max, coeff_dtype, False)[1:]


@_compute_coeffs_op.register_fake
def _(dyn, rw, x_conv, mask, dtb, rlog, wlog, ltau, H, R, M, read_temp, dt_min, dt_max, alpha_min, alpha_max,
      lambda_min, lambda_max, coeff_dtype):
    B, L, _ = x_conv.shape
    dev = x_conv.device
    c = torch.empty(B * H, L, M, device=dev, dtype=coeff_dtype)
    return c, torch.empty_like(c), torch.empty(B * H, L, M, device=dev, dtype=torch.float32)


def frac_compute_scan_params(model, x_conv, x, attention_mask=None):
    """Compute scan inputs (u, c, kappa, rho) from post-conv features.

    `model` is a mixer holding dyn_proj, rw_proj, dt_bias, read_residual_logit,
    write_residual_scale, base_log_tau, num_heads, head_dim, num_modes, read_temp and config.
    """
    dyn = F.linear(x, model.dyn_proj.weight, model.dyn_proj.bias)
    rw = F.linear(x_conv, model.rw_proj.weight)
    cfg = model.config
    return compute_params_from_projections(
        dyn, rw, x_conv, attention_mask, model.dt_bias, model.read_residual_logit,
        model.write_residual_scale, model.base_log_tau, model.num_heads, model.head_dim,
        model.num_modes, model.read_temp, cfg.frac_dt_min, cfg.frac_dt_max, cfg.frac_alpha_min,
        cfg.frac_alpha_max, cfg.frac_lambda_min, cfg.frac_lambda_max)
