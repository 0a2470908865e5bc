"""D skip connection + un-flatten on the B200 CUDA extension
(interface of `frac_ssm/layers/output_mix.py:232-243`), and the fused epilogue that also
applies the gated RMSNorm (`frac_ssm/models/modeling_frac.py:213-214`).  Forward only."""

import torch

from .. import _cabi as C
from ..ops.b200.stages import _op


def skip_mix(mixed_flat, x_conv, D, num_heads, head_dim, out_dtype=None):
    """out[b, l, h*R + r] = mixed_flat[b*H + h, l, r] + x_conv[b, l, h*R + r] * D[h, r]."""
    assert mixed_flat.dim() == 3 and x_conv.dim() == 3, "mixed_flat and x_conv must be 3D"
    assert mixed_flat.is_cuda and x_conv.is_cuda, "inputs must be on CUDA"
    H, R = num_heads, head_dim
    B, L, HR = x_conv.shape
    assert HR == H * R, "x_conv last dim must be num_heads * head_dim"
    assert mixed_flat.shape == (B * H, L, R), "mixed_flat shape must be (B*H, L, R)"
    out_dtype = x_conv.dtype if out_dtype is None else out_dtype
    Df = D.detach().to(device=x_conv.device, dtype=torch.float32).contiguous()
    return _skip_mix_op(mixed_flat, x_conv, Df, H, R, out_dtype)


# the launches below are torch custom ops with shape-only implementations (torch.compile(fullgraph=True))
@_op("skip_mix")
def _skip_mix_op(mixed_flat: torch.Tensor, x_conv: torch.Tensor, Df: torch.Tensor, H: int, R: int,
                 out_dtype: torch.dtype) -> torch.Tensor:
    B, L, HR = x_conv.shape
    mixed_flat, x_conv = C.rows(mixed_flat), C.rows(x_conv)
    out = torch.empty(B, L, HR, device=x_conv.device, dtype=out_dtype)
    if B == 0 or L == 0:
        return out
    with C.trace("frac_skip_mix"), torch.cuda.device(x_conv.device):
        C.check(C.lib().fracssm_skip_mix(
            C.ptr(mixed_flat), C.dt(mixed_flat), mixed_flat.stride(0), mixed_flat.stride(1),
            C.ptr(x_conv), C.dt(x_conv), x_conv.stride(0), x_conv.stride(1), C.ptr(Df), C.ptr(out),
            C.dt(out), B, L, H, R, C.stream_of(x_conv)), "skip_mix")
    return out


@_skip_mix_op.register_fake
def _(mixed_flat, x_conv, Df, H, R, out_dtype):
    return torch.empty(x_conv.shape, device=x_conv.device, dtype=out_dtype)


def frac_skip_mix(model, mixed_flat, x_conv, out_dtype=None):
    """D skip connection, reshape."""
    return skip_mix(mixed_flat, x_conv, model.D, model.num_heads, model.head_dim, out_dtype)


def scan_epilogue(h, x_conv, gate, D, weight, num_heads, head_dim, eps=1e-6, gate_bias=0.0):
    """y = weight * rmsnorm((h_unflat + x_conv * D) * silu(gate + gate_bias)) in one pass."""
    assert h.dim() == 3 and x_conv.dim() == 3 and gate.dim() == 3, "h, x_conv and gate must be 3D"
    assert h.is_cuda and x_conv.is_cuda and gate.is_cuda, "inputs must be on CUDA"
    H, R = num_heads, head_dim
    B, L, HR = x_conv.shape
    assert HR == H * R and gate.shape == x_conv.shape and h.shape == (B * H, L, R)
    assert gate.dtype == x_conv.dtype, "gate and x_conv must have the same dtype"
    Df = D.detach().to(device=x_conv.device, dtype=torch.float32).contiguous()
    return _scan_epilogue_op(h, x_conv, gate, Df, weight.detach().contiguous(), H, R, float(eps), float(gate_bias))


@_op("scan_epilogue")
def _scan_epilogue_op(h: torch.Tensor, x_conv: torch.Tensor, gate: torch.Tensor, Df: torch.Tensor, w: torch.Tensor,
                      H: int, R: int, eps: float, gate_bias: float) -> torch.Tensor:
    B, L, HR = x_conv.shape
    h, x_conv, gate = C.rows(h), C.rows(x_conv), C.rows(gate)
    y = torch.empty(B, L, HR, device=x_conv.device, dtype=x_conv.dtype)
    if B == 0 or L == 0:
        return y
    with C.trace("scan_epilogue"), torch.cuda.device(x_conv.device):
        C.check(C.lib().fracssm_scan_epilogue(
            C.ptr(h), C.dt(h), h.stride(0), h.stride(1), C.ptr(x_conv), x_conv.stride(0),
            x_conv.stride(1), C.ptr(gate), gate.stride(0), gate.stride(1), C.dt(x_conv), C.ptr(Df),
            C.ptr(w), C.dt(w), float(gate_bias), float(eps), C.ptr(y), B, L, H, R,
            C.stream_of(x_conv)), "scan_epilogue")
    return y


@_scan_epilogue_op.register_fake
def _(h, x_conv, gate, Df, w, H, R, eps, gate_bias):
    return torch.empty_like(x_conv)


def _epilogue_args(h, x_conv, gate, D, num_heads, head_dim):
    assert h.dim() == 3 and x_conv.dim() == 3 and gate.dim() == 3, "h, x_conv and gate must be 3D"
    assert h.is_cuda and x_conv.is_cuda and gate.is_cuda, "inputs must be on CUDA"
    H, R = num_heads, head_dim
    B, L, HR = x_conv.shape
    assert HR == H * R and gate.shape == x_conv.shape and h.shape == (B * H, L, R)
    assert gate.dtype == x_conv.dtype, "gate and x_conv must have the same dtype"
    Df = D.detach().to(device=x_conv.device, dtype=torch.float32).contiguous()
    return C.rows(h), C.rows(x_conv), C.rows(gate), Df, B, L, H, R


def scan_epilogue_sumsq(h, x_conv, gate, D, num_heads, head_dim, gate_bias=0.0):
    """First pass of the epilogue of a head-sharded layer: per (b, l) row, the sum of squares of
    (h_unflat + x_conv * D) * silu(gate + gate_bias) over the local heads, float32 [B, L]."""
    h, x_conv, gate, Df, B, L, H, R = _epilogue_args(h, x_conv, gate, D, num_heads, head_dim)
    sumsq = torch.zeros(B, L, device=x_conv.device, dtype=torch.float32)
    if B == 0 or L == 0:
        return sumsq
    with torch.cuda.device(x_conv.device):
        C.check(C.lib().fracssm_scan_epilogue_sumsq(
            C.ptr(h), C.dt(h), h.stride(0), h.stride(1), C.ptr(x_conv), x_conv.stride(0),
            x_conv.stride(1), C.ptr(gate), gate.stride(0), gate.stride(1), C.dt(x_conv), C.ptr(Df),
            float(gate_bias), C.ptr(sumsq), B, L, H, R, C.stream_of(x_conv)), "scan_epilogue_sumsq")
    return sumsq


def scan_epilogue_apply(h, x_conv, gate, D, weight, num_heads, head_dim, sumsq, norm_width, eps=1e-6,
                        gate_bias=0.0):
    """Second pass: the local columns normalised with `sumsq` [B, L], the rows' sums of squares over
    all `norm_width` columns of the layer (the first pass's result added across GPUs)."""
    h, x_conv, gate, Df, B, L, H, R = _epilogue_args(h, x_conv, gate, D, num_heads, head_dim)
    assert sumsq.shape == (B, L) and sumsq.dtype == torch.float32 and sumsq.is_cuda
    assert norm_width >= H * R, "norm_width is the layer's full width"
    w = weight.detach().contiguous()
    assert w.numel() == H * R, "weight holds the local columns"
    sumsq = sumsq.contiguous()
    y = torch.empty(B, L, H * R, device=x_conv.device, dtype=x_conv.dtype)
    if B == 0 or L == 0:
        return y
    with torch.cuda.device(x_conv.device):
        C.check(C.lib().fracssm_scan_epilogue_apply(
            C.ptr(h), C.dt(h), h.stride(0), h.stride(1), C.ptr(x_conv), x_conv.stride(0),
            x_conv.stride(1), C.ptr(gate), gate.stride(0), gate.stride(1), C.dt(x_conv), C.ptr(Df),
            C.ptr(w), C.dt(w), float(gate_bias), float(eps), C.ptr(sumsq), int(norm_width), C.ptr(y),
            B, L, H, R, C.stream_of(x_conv)), "scan_epilogue_apply")
    return y


def scan_layer_supported(u, c, gate) -> bool:
    """True when the fused layer path (scan + skip-mix + gate in one kernel) covers these tensors."""
    return (u.is_cuda and u.dtype == torch.bfloat16 and gate.dtype == torch.bfloat16 and u.dim() == 3
            and u.shape[-1] == 64 and c.shape[-1] == 128 and c.dtype in (torch.bfloat16, torch.float32)
            and u.shape[0] > 0 and u.shape[1] > 0)


def scan_layer_gated(u, c, kappa, rho, gate, D, num_heads, gate_bias=0.0, initial_state=None,
                     return_final_state=False, final_state_dtype=torch.float32):
    """First pass of the fused layer path: the scan with the skip connection and the gate applied in
    its output stage.  Returns (gated [batch, L, H*64] bf16, ss_partial [batch, L, H, 4] float32,
    final_state or None); h itself is never written."""
    assert scan_layer_supported(u, c, gate), "scan_layer needs CUDA bf16 u / gate with R = 64, M = 128"
    assert rho.dtype == torch.float32, "rho must be float32 for numerical stability"
    BH, L, R = u.shape
    M = c.shape[-1]
    H = num_heads
    assert BH % H == 0 and gate.shape == (BH // H, L, H * R), "gate must be [batch, L, num_heads * head_dim]"
    Bt = BH // H
    u, c, kappa, rho, gate = (t.contiguous() for t in (u, c, kappa, rho, gate))
    init = None if initial_state is None else initial_state.contiguous()
    Df = D.detach().to(device=u.device, dtype=torch.float32).contiguous()
    gated = torch.empty(Bt, L, H * R, device=u.device, dtype=torch.bfloat16)
    ss = torch.empty(Bt, L, H, 4, device=u.device, dtype=torch.float32)
    fin = torch.empty(BH, R, M, device=u.device, dtype=final_state_dtype) if return_final_state else None
    lib = C.lib()
    with C.trace("scan_layer_gated"), torch.cuda.device(u.device):
        ws = torch.empty(max(lib.fracssm_scan_layer_workspace_bytes(Bt, H, L, R, M), 256), device=u.device,
                         dtype=torch.uint8)
        C.check(lib.fracssm_scan_layer_gated(
            C.ptr(u), C.ptr(c), C.ptr(kappa), C.dt(c), C.ptr(rho), C.ptr(init), C.ptr(gate), C.ptr(Df),
            float(gate_bias), C.ptr(gated), C.ptr(ss), C.ptr(fin), C.dt_of(final_state_dtype), C.ptr(ws),
            ws.numel(), Bt, H, L, R, M, C.stream_of(u)), "scan_layer_gated")
    return gated, ss, fin


def scan_layer_sumsq(ss_partial):
    """Per (b, l) row, the sum of the partial sums of squares of the local heads: float32 [batch, L]."""
    Bt, L, H, _ = ss_partial.shape
    out = torch.empty(Bt, L, device=ss_partial.device, dtype=torch.float32)
    with torch.cuda.device(ss_partial.device):
        C.check(C.lib().fracssm_scan_layer_sumsq(C.ptr(ss_partial), C.ptr(out), Bt, L, H,
                                                 C.stream_of(ss_partial)), "scan_layer_sumsq")
    return out


def scan_layer_norm(gated, ss_partial, weight, head_dim, eps=1e-6, sumsq=None, norm_width=None):
    """Second pass: y = weight * gated * rsqrt(mean(gated^2) + eps) per row; `sumsq` / `norm_width`
    override the row total and the width when the layer's heads are spread over several GPUs."""
    Bt, L, HR = gated.shape
    H = HR // head_dim
    w = weight.detach().contiguous()
    y = torch.empty_like(gated)
    with C.trace("scan_layer_norm"), torch.cuda.device(gated.device):
        C.check(C.lib().fracssm_scan_layer_norm(
            C.ptr(gated), C.ptr(ss_partial), C.ptr(sumsq), C.ptr(w), C.dt(w), float(eps),
            int(HR if norm_width is None else norm_width), C.ptr(y), Bt, L, H, head_dim,
            C.stream_of(gated)), "scan_layer_norm")
    return y


def scan_layer(u, c, kappa, rho, gate, D, weight, num_heads, eps=1e-6, gate_bias=0.0, initial_state=None,
               return_final_state=False, final_state_dtype=torch.float32):
    """frac_scan -> frac_skip_mix -> gated RMSNorm of one layer in two kernels, without writing h
    (`frac_ssm/models/modeling_frac.py:203-214`).  u [batch*H, L, 64] is the head-major copy of x_conv."""
    gated, ss, fin = scan_layer_gated(u, c, kappa, rho, gate, D, num_heads, gate_bias, initial_state,
                                      return_final_state, final_state_dtype)
    y = scan_layer_norm(gated, ss, weight, u.shape[-1], eps)
    return (y, fin) if return_final_state else y
