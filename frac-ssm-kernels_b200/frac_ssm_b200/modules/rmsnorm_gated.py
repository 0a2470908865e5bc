"""Gated RMSNorm on the B200 CUDA extension (interface of
`frac_ssm/modules/rmsnorm_gated.py:65-99,292-299`).  Forward only."""

from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import _cabi as C
from ..ops.b200.stages import _op


def rmsnorm_gated_fwd(hidden_states, weight, gate=None, eps=1e-6):
    """One-pass RMSNorm forward with optional gating (before the norm) -> (output, rstd)."""
    assert hidden_states.is_cuda, "hidden_states must be on CUDA"
    shape = hidden_states.shape
    D = shape[-1]
    x = hidden_states.reshape(-1, D)
    if x.stride(-1) != 1:
        x = x.contiguous()
    g = None
    if gate is not None:
        assert gate.shape == shape and gate.dtype == hidden_states.dtype, (
            "gate must match hidden_states in shape and dtype")
        g = gate.reshape(-1, D)
        if g.stride(-1) != 1:
            g = g.contiguous()
    w = weight.detach().contiguous()
    assert w.numel() == D, "weight must have hidden_size elements"
    y, rstd = _rmsnorm_gated_op(x, g, w, float(eps))
    return y.reshape(shape), rstd.reshape(shape[:-1])


# a torch custom op with a shape-only implementation, so the norm can sit inside torch.compile(fullgraph=True)
@_op("rmsnorm_gated")
def _rmsnorm_gated_op(x: torch.Tensor, g: Optional[torch.Tensor], w: torch.Tensor,
                      eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    rows, D = x.shape
    y = torch.empty(rows, D, device=x.device, dtype=x.dtype)
    rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
    if rows > 0:
        with C.trace("rmsnorm_gated"), torch.cuda.device(x.device):
            C.check(C.lib().fracssm_rmsnorm_gated(
                C.ptr(x), x.stride(0), C.ptr(g), 0 if g is None else g.stride(0), C.dt(x), C.ptr(w),
                C.dt(w), float(eps), C.ptr(y), C.ptr(rstd), rows, D, C.stream_of(x)), "rmsnorm_gated")
    return y, rstd


@_rmsnorm_gated_op.register_fake
def _(x, g, w, eps):
    return torch.empty_like(x), torch.empty(x.shape[0], device=x.device, dtype=torch.float32)


class MambaRMSNormGated(nn.Module):
    def __init__(self, hidden_size, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, hidden_states, gate=None):
        return rmsnorm_gated_fwd(hidden_states, self.weight, gate, self.variance_epsilon)[0]
