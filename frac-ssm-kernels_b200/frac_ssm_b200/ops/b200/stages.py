"""Per-stage forward ops of the chunked scan on the B200 CUDA extension.

Same names, argument order, defaults and assertion messages as the per-stage entry points
of quorbix/frac-ssm-kernels (`frac_ssm/ops/triton/chunk_cumsum.py:189`,
`chunk_state.py:305`, `state_passing.py:322`, `chunk_w.py:418`, `chunk_readout.py:657`,
`frac_ssm/ops/cute/chunk_fused_readout.py:150`).  Forward only; inputs are never modified,
outputs are freshly allocated on the input device, kernels run on the current stream.
"""

from typing import Optional, Tuple

import torch

from ... import _cabi as C

# Every launch below is a torch custom op with a shape-only "fake" implementation, so the stage ops
# can sit inside torch.compile(fullgraph=True) as the reference's do
# (frac_ssm/ops/triton/chunk_state.py:243-302).  Forward only: asking for gradients raises.


def _no_backward(ctx, *grads):
    raise NotImplementedError("frac_ssm_b200 implements the forward pass only")


def _op(name):
    def wrap(fn):
        op = torch.library.custom_op(f"frac_ssm_b200::{name}", mutates_args=())(fn)
        op.register_autograd(_no_backward)
        return op
    return wrap


def _nchunks(L: int, T: int) -> int:
    return (L + T - 1) // T


def chunk_cumsum(log_rho, chunk_size):
    """Per-chunk inclusive running sum of log_rho -> (log_cum_rho [B,L,M], chunk_decay [B,N,M])."""
    assert log_rho.dim() == 3, f"log_rho must be 3D (B, L, M), got {log_rho.dim()}D"
    assert log_rho.is_cuda, "log_rho must be on CUDA"
    assert log_rho.dtype == torch.float32, f"log_rho dtype must be float32, got {log_rho.dtype}"
    assert (
        isinstance(chunk_size, int) and chunk_size > 0 and (chunk_size & (chunk_size - 1)) == 0
    ), f"chunk_size must be a positive power of two, got {chunk_size}"
    return _cumsum(log_rho, chunk_size, False)


def _cumsum(src, chunk_size, src_is_rho):
    lcr, cd = _cumsum_op(src, chunk_size, bool(src_is_rho))
    return lcr, cd


@_op("chunk_cumsum")
def _cumsum_op(src: torch.Tensor, chunk_size: int, src_is_rho: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    B, L, M = src.shape
    N = _nchunks(L, chunk_size)
    src = C.rows(src)
    lcr = torch.empty(B, L, M, device=src.device, dtype=torch.float32)
    cd = torch.empty(B, N, M, device=src.device, dtype=torch.float32)
    if B == 0 or L == 0:
        return lcr, cd
    with torch.cuda.device(src.device):
        C.check(C.lib().fracssm_chunk_cumsum(C.ptr(src), src.stride(0), src.stride(1), int(src_is_rho),
                                             C.ptr(lcr), C.ptr(cd), B, L, M, chunk_size,
                                             C.stream_of(src)), "chunk_cumsum")
    return lcr, cd


@_cumsum_op.register_fake
def _(src, chunk_size, src_is_rho):
    B, L, M = src.shape
    return (torch.empty(B, L, M, device=src.device, dtype=torch.float32),
            torch.empty(B, _nchunks(L, chunk_size), M, device=src.device, dtype=torch.float32))


def chunk_state(u, kappa, log_cum_rho, chunk_size, state_fp32=True):
    """Per-chunk state contribution -> states [B, N, R, M] (float32, or u.dtype if not state_fp32)."""
    assert u.dim() == 3, f"u must be 3D (B, L, R), got {u.dim()}D"
    assert kappa.dim() == 3, f"kappa must be 3D (B, L, M), got {kappa.dim()}D"
    assert log_cum_rho.dim() == 3, f"log_cum_rho must be 3D (B, L, M), got {log_cum_rho.dim()}D"
    assert u.is_cuda and kappa.is_cuda and log_cum_rho.is_cuda, "inputs must be on CUDA"
    assert log_cum_rho.dtype == torch.float32, (
        f"log_cum_rho dtype must be float32, got {log_cum_rho.dtype}"
    )
    assert chunk_size > 0, f"chunk_size must be positive, got {chunk_size}"
    B, L, R = u.shape
    M = kappa.shape[-1]
    N = _nchunks(L, chunk_size)
    sdt = torch.float32 if state_fp32 else u.dtype
    assert sdt in (torch.float32, torch.bfloat16), f"states dtype must be float32 or bfloat16, got {sdt}"
    return _chunk_state_op(u, kappa, log_cum_rho, chunk_size, sdt == torch.float32)


@_op("chunk_state")
def _chunk_state_op(u: torch.Tensor, kappa: torch.Tensor, log_cum_rho: torch.Tensor, chunk_size: int,
                    fp32: bool) -> torch.Tensor:
    B, L, R = u.shape
    M = kappa.shape[-1]
    N = _nchunks(L, chunk_size)
    u, kappa, g = C.rows(u), C.rows(kappa), C.rows(log_cum_rho)
    states = torch.empty(B, N, R, M, device=u.device, dtype=torch.float32 if fp32 else torch.bfloat16)
    if B == 0 or L == 0:
        return states
    with torch.cuda.device(u.device):
        C.check(C.lib().fracssm_chunk_state(
            C.ptr(u), C.dt(u), u.stride(0), u.stride(1), C.ptr(kappa), C.dt(kappa), kappa.stride(0),
            kappa.stride(1), C.ptr(g), g.stride(0), g.stride(1), C.ptr(states), C.dt(states),
            B, L, R, M, chunk_size, C.stream_of(u)), "chunk_state")
    return states


@_chunk_state_op.register_fake
def _(u, kappa, log_cum_rho, chunk_size, fp32):
    B, L, R = u.shape
    return torch.empty(B, _nchunks(L, chunk_size), R, kappa.shape[-1], device=u.device,
                       dtype=torch.float32 if fp32 else torch.bfloat16)


def state_passing(states, chunk_decay, initial_state=None):
    """Inter-chunk recurrence -> (states_acc [B,N,R,M], final_state [B,R,M]), both in states.dtype."""
    assert states.dim() == 4, f"states must be 4D (B, N, R, M), got {states.dim()}D"
    assert chunk_decay.dim() == 3, f"chunk_decay must be 3D (B, N, M), got {chunk_decay.dim()}D"
    assert states.is_cuda and chunk_decay.is_cuda, "states and chunk_decay must be on CUDA"
    assert states.dtype in (torch.float32, torch.bfloat16), (
        f"states dtype must be float32 or bfloat16, got {states.dtype}"
    )
    assert chunk_decay.dtype == torch.float32, (
        f"chunk_decay dtype must be float32, got {chunk_decay.dtype}"
    )
    if initial_state is not None:
        assert initial_state.dim() == 3, (
            f"initial_state must be 3D (B, R, M), got {initial_state.dim()}D"
        )
        assert initial_state.is_cuda, "initial_state must be on CUDA"
        assert initial_state.dtype in (torch.float32, torch.bfloat16), (
            f"initial_state dtype must be float32 or bfloat16, got {initial_state.dtype}"
        )
    return _state_passing(states, chunk_decay, initial_state, states.dtype, states.dtype)


def _state_passing(states, chunk_decay, initial_state, acc_dtype, final_dtype):
    acc, fin = _state_passing_op(states, chunk_decay, initial_state, acc_dtype == torch.float32,
                                 final_dtype == torch.float32)
    return acc, fin


@_op("state_passing")
def _state_passing_op(states: torch.Tensor, chunk_decay: torch.Tensor, initial_state: Optional[torch.Tensor],
                      acc_fp32: bool, final_fp32: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    acc_dtype = torch.float32 if acc_fp32 else torch.bfloat16
    final_dtype = torch.float32 if final_fp32 else torch.bfloat16
    B, N, R, M = states.shape
    states, chunk_decay = states.contiguous(), chunk_decay.contiguous()
    init = None if initial_state is None else initial_state.contiguous()
    acc = torch.empty(B, N, R, M, device=states.device, dtype=acc_dtype)
    fin = torch.empty(B, R, M, device=states.device, dtype=final_dtype)
    if B == 0:
        return acc, fin
    with torch.cuda.device(states.device):
        C.check(C.lib().fracssm_state_passing(
            C.ptr(states), C.dt(states), C.ptr(chunk_decay), C.ptr(init),
            C.F32 if init is None else C.dt(init), C.ptr(acc), C.dt(acc), C.ptr(fin), C.dt(fin),
            B, N, R, M, C.stream_of(states)), "state_passing")
    return acc, fin


@_state_passing_op.register_fake
def _(states, chunk_decay, initial_state, acc_fp32, final_fp32):
    B, N, R, M = states.shape
    return (torch.empty(B, N, R, M, device=states.device, dtype=torch.float32 if acc_fp32 else torch.bfloat16),
            torch.empty(B, R, M, device=states.device, dtype=torch.float32 if final_fp32 else torch.bfloat16))


def chunk_w(c, kappa, log_cum_rho, chunk_size):
    """Causal per-chunk interaction matrix W [B, N, T, T] (float32)."""
    assert c.dim() == 3, f"c must be 3D (B, L, M), got {c.dim()}D"
    assert kappa.dim() == 3, f"kappa must be 3D (B, L, M), got {kappa.dim()}D"
    assert log_cum_rho.dim() == 3, (
        f"log_cum_rho must be 3D (B, L, M), got {log_cum_rho.dim()}D"
    )
    assert c.is_cuda and kappa.is_cuda and log_cum_rho.is_cuda, "inputs must be on CUDA"
    assert c.dtype == kappa.dtype, (
        f"c and kappa must have the same dtype, got {c.dtype} and {kappa.dtype}"
    )
    assert c.dtype in (torch.float32, torch.bfloat16), (
        f"c and kappa dtype must be float32 or bfloat16, got {c.dtype}"
    )
    assert log_cum_rho.dtype == torch.float32, (
        f"log_cum_rho dtype must be float32, got {log_cum_rho.dtype}"
    )
    M = c.shape[-1]
    assert M > 0 and (M & (M - 1)) == 0, f"M must be a positive power of two, got {M}"
    assert chunk_size > 0 and chunk_size % 32 == 0, (
        f"chunk_size must be a positive multiple of 32, got {chunk_size}"
    )
    return _chunk_w_op(c, kappa, log_cum_rho, chunk_size)


@_op("chunk_w")
def _chunk_w_op(c: torch.Tensor, kappa: torch.Tensor, log_cum_rho: torch.Tensor, chunk_size: int) -> torch.Tensor:
    M = c.shape[-1]
    B, L, _ = log_cum_rho.shape
    N = _nchunks(L, chunk_size)
    c, kappa, g = C.rows(c), C.rows(kappa), C.rows(log_cum_rho)
    W = torch.empty(B, N, chunk_size, chunk_size, device=c.device, dtype=torch.float32)
    if B == 0 or L == 0:
        return W
    with torch.cuda.device(c.device):
        C.check(C.lib().fracssm_chunk_w(
            C.ptr(c), C.ptr(kappa), C.dt(c), c.stride(0), c.stride(1), kappa.stride(0),
            kappa.stride(1), C.ptr(g), g.stride(0), g.stride(1), C.ptr(W), B, L, M, chunk_size,
            C.stream_of(c)), "chunk_w")
    return W


@_chunk_w_op.register_fake
def _(c, kappa, log_cum_rho, chunk_size):
    B, L, _ = log_cum_rho.shape
    return torch.empty(B, _nchunks(L, chunk_size), chunk_size, chunk_size, device=c.device, dtype=torch.float32)


def chunk_readout(u, c, states_acc, W, log_cum_rho, chunk_size):
    """Apply the carried-state and intra-chunk contributions -> h [B, L, R] in u.dtype."""
    assert u.dim() == 3, f"u must be 3D (B, L, R), got {u.dim()}D"
    assert c.dim() == 3, f"c must be 3D (B, L, M), got {c.dim()}D"
    assert states_acc.dim() == 4, f"states_acc must be 4D (B, N, R, M), got {states_acc.dim()}D"
    assert W.dim() == 4, f"W must be 4D (B, N, C, C), got {W.dim()}D"
    assert log_cum_rho.dim() == 3, f"log_cum_rho must be 3D (B, L, M), got {log_cum_rho.dim()}D"
    assert all(x.is_cuda for x in (u, c, states_acc, W, log_cum_rho)), "inputs must be on CUDA"
    assert states_acc.dtype in (u.dtype, torch.float32), (
        f"states_acc dtype must be {u.dtype} or float32, got {states_acc.dtype}"
    )
    assert W.dtype in (u.dtype, torch.float32), (
        f"W dtype must be {u.dtype} or float32, got {W.dtype}"
    )
    assert log_cum_rho.dtype == torch.float32, (
        f"log_cum_rho dtype must be float32, got {log_cum_rho.dtype}"
    )
    assert chunk_size > 0, f"chunk_size must be positive, got {chunk_size}"
    B, L, R = u.shape
    M = c.shape[-1]
    N = _nchunks(L, chunk_size)
    assert c.shape == (B, L, M), "c shape must be (B, L, M)"
    assert log_cum_rho.shape == (B, L, M), "log_cum_rho shape must be (B, L, M)"
    assert states_acc.shape == (B, N, R, M), "states_acc shape must be (B, nchunks, R, M)"
    assert W.shape == (B, N, chunk_size, chunk_size), (
        "W shape must be (B, nchunks, chunk_size, chunk_size)"
    )
    return _chunk_readout_op(u, c, states_acc, W, log_cum_rho, chunk_size)


@_op("chunk_readout")
def _chunk_readout_op(u: torch.Tensor, c: torch.Tensor, states_acc: torch.Tensor, W: torch.Tensor,
                      log_cum_rho: torch.Tensor, chunk_size: int) -> torch.Tensor:
    B, L, R = u.shape
    M = c.shape[-1]
    u, c, g = C.rows(u), C.rows(c), C.rows(log_cum_rho)
    states_acc, W = states_acc.contiguous(), W.contiguous()
    h = torch.empty(B, L, R, device=u.device, dtype=u.dtype)
    if B == 0 or L == 0:
        return h
    with torch.cuda.device(u.device):
        C.check(C.lib().fracssm_chunk_readout(
            C.ptr(u), C.dt(u), u.stride(0), u.stride(1), C.ptr(c), C.dt(c), c.stride(0), c.stride(1),
            C.ptr(states_acc), C.dt(states_acc), C.ptr(W), C.dt(W), C.ptr(g), g.stride(0),
            g.stride(1), C.ptr(h), B, L, R, M, chunk_size, C.stream_of(u)), "chunk_readout")
    return h


@_chunk_readout_op.register_fake
def _(u, c, states_acc, W, log_cum_rho, chunk_size):
    return torch.empty_like(u)


def chunk_fused_readout(u, c, kappa, states_acc, log_cum_rho, chunk_size):
    """chunk_w and chunk_readout in one kernel (W is never stored) -> h [B, L, R] in u.dtype."""
    assert u.dim() == 3, f"u must be 3D (B, L, R), got {u.dim()}D"
    assert c.dim() == 3, f"c must be 3D (B, L, M), got {c.dim()}D"
    assert kappa.dim() == 3, f"kappa must be 3D (B, L, M), got {kappa.dim()}D"
    assert states_acc.dim() == 4, f"states_acc must be 4D (B, N, R, M), got {states_acc.dim()}D"
    assert log_cum_rho.dim() == 3, f"log_cum_rho must be 3D (B, L, M), got {log_cum_rho.dim()}D"
    assert all(x.is_cuda for x in (u, c, kappa, states_acc, log_cum_rho)), "inputs must be on CUDA"
    assert c.dtype == kappa.dtype and c.dtype in (u.dtype, torch.float32), (
        "c and kappa dtype must match u dtype or be float32"
    )
    assert states_acc.dtype in (u.dtype, torch.float32), (
        f"states_acc dtype must be {u.dtype} or float32, got {states_acc.dtype}"
    )
    assert log_cum_rho.dtype == torch.float32, (
        f"log_cum_rho dtype must be float32, got {log_cum_rho.dtype}"
    )
    assert isinstance(chunk_size, int) and chunk_size > 0, (
        f"chunk_size must be a positive integer, got {chunk_size}"
    )
    B, L, R = u.shape
    M = c.shape[-1]
    N = _nchunks(L, chunk_size)
    assert c.shape == (B, L, M) and kappa.shape == (B, L, M), "c and kappa shapes must match (B, L, M)"
    assert log_cum_rho.shape == (B, L, M), "log_cum_rho shape must match (B, L, M)"
    assert states_acc.shape == (B, N, R, M), "states_acc shape must be (B, nchunks, R, M)"
    return _chunk_fused_readout_op(u, c, kappa, states_acc, log_cum_rho, chunk_size)


@_op("chunk_fused_readout")
def _chunk_fused_readout_op(u: torch.Tensor, c: torch.Tensor, kappa: torch.Tensor, states_acc: torch.Tensor,
                            log_cum_rho: torch.Tensor, chunk_size: int) -> torch.Tensor:
    B, L, R = u.shape
    M = c.shape[-1]
    u, c, kappa, g = C.rows(u), C.rows(c), C.rows(kappa), C.rows(log_cum_rho)
    states_acc = states_acc.contiguous()
    h = torch.empty(B, L, R, device=u.device, dtype=u.dtype)
    if B == 0 or L == 0:
        return h
    with torch.cuda.device(u.device):
        C.check(C.lib().fracssm_chunk_fused_readout(
            C.ptr(u), C.dt(u), u.stride(0), u.stride(1), C.ptr(c), C.ptr(kappa), C.dt(c),
            c.stride(0), c.stride(1), kappa.stride(0), kappa.stride(1), C.ptr(states_acc),
            C.dt(states_acc), C.ptr(g), g.stride(0), g.stride(1), C.ptr(h), B, L, R, M, chunk_size,
            C.stream_of(u)), "chunk_fused_readout")
    return h


@_chunk_fused_readout_op.register_fake
def _(u, c, kappa, states_acc, log_cum_rho, chunk_size):
    return torch.empty_like(u)


__all__ = ["chunk_cumsum", "chunk_state", "state_passing", "chunk_w", "chunk_readout",
           "chunk_fused_readout"]
