"""The composed forward scan on the B200 CUDA extension.

Backend-module interface of the reference (`frac_ssm/ops/triton/frac_scan.py:102-130`):
`frac_scan(u, c, kappa, rho, chunk_size, initial_state=None, return_final_state=False)`.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from ... import _cabi as C

# "auto": the single-pass tcgen05 kernel when it covers the shape, else the staged kernels.
_PATHS = {"auto": C.PATH_AUTO, "staged": C.PATH_STAGED, "fused": C.PATH_FUSED}

def frac_scan(u, c, kappa, rho, chunk_size, initial_state=None, return_final_state=False, *,
              final_state_dtype=None, path="auto", check=False):
    """Fractional chunked scan, forward.

    Args:
        u: [B, L, R] input features (bfloat16, float16 or float32); dim 0 is batch*heads.
        c, kappa: [B, L, M] read / write coefficients, same dtype as each other (u's or float32).
        rho: [B, L, M] float32 decay.
        chunk_size: tokens per chunk.
        initial_state: [B, R, M] float32 or None.
        return_final_state: also return the state after the last token.
        final_state_dtype: dtype of the returned state; default follows the reference
            (bfloat16 when u is bfloat16, else float32).  The state is always carried in float32.
        path: "auto", "staged" or "fused".  "auto" takes the single-pass kernel when it covers the
            shape, and for few rows with many tokens (at most 28 rows, at least 32768 tokens) cuts
            every row into sub-segments first, because a row is one chain of tiles and 148 SMs want
            more chains than that: one summary pass over u, kappa and rho gives every sub-segment its
            incoming state, then all sub-segments are scanned as rows (`parallel.seq_parallel_scan`).
        check: after the launch, synchronise and raise if a bounded device-side wait of the
            single-pass kernel ran out (debugging aid; the default stays asynchronous).
    Returns:
        h [B, L, R] in u.dtype, and final_state [B, R, M] if requested.
    """
    assert rho.dtype == torch.float32, "rho must be float32 for numerical stability"
    if initial_state is not None:
        assert initial_state.dtype == torch.float32, "initial_state must be float32"
    assert u.dim() == 3, f"u must be 3D (B, L, R), got {u.dim()}D"
    assert c.dim() == 3, f"c must be 3D (B, L, M), got {c.dim()}D"
    assert kappa.dim() == 3, f"kappa must be 3D (B, L, M), got {kappa.dim()}D"
    assert rho.dim() == 3, f"rho must be 3D (B, L, M), got {rho.dim()}D"
    assert all(x.is_cuda for x in (u, c, kappa, rho)), "inputs must be on CUDA"
    assert c.dtype == kappa.dtype and c.dtype in (u.dtype, torch.float32), (
        "c and kappa dtype must match u dtype or be float32"
    )
    assert isinstance(chunk_size, int) and chunk_size > 0, (
        f"chunk_size must be a positive integer, got {chunk_size}"
    )
    B, L, R = u.shape
    M = c.shape[-1]
    assert c.shape == (B, L, M) and kappa.shape == (B, L, M) and rho.shape == (B, L, M), (
        "c, kappa and rho shapes must match (B, L, M)"
    )
    if initial_state is not None:
        assert initial_state.shape == (B, R, M), "initial_state shape must be (B, R, M)"
        assert initial_state.is_cuda, "initial_state must be on CUDA"
    if final_state_dtype is None:
        final_state_dtype = torch.bfloat16 if u.dtype == torch.bfloat16 else torch.float32
    assert final_state_dtype in (torch.float32, torch.bfloat16)

    path_code = _PATHS[path]
    if path == "auto" and not check and not torch.compiler.is_compiling():
        splits = _row_splits(u, c, chunk_size)
        if splits > 1:
            from ... import parallel
            h, fin = parallel.seq_parallel_scan(u, c, kappa, rho, chunk_size, initial_state, True,
                                                local_splits=splits, process_local=True)
            return (h, fin.to(final_state_dtype)) if return_final_state else h
    if check:      # the status read-back bypasses the registered op (it needs the scratch)
        h, fin = _launch(u, c, kappa, rho, chunk_size, initial_state, return_final_state,
                         final_state_dtype == torch.float32, path_code, check)
    else:
        h, fin = _frac_scan_fwd_op(u, c, kappa, rho, chunk_size, initial_state, return_final_state,
                                   final_state_dtype == torch.float32, path_code)
    if return_final_state:
        return h, fin
    return h


def _row_splits(u, c, chunk_size):
    """Sub-segments per row for the "auto" path: more than 1 only where the single-pass kernel covers
    both the call and the cut-up call, the tensors are dense, and the rows are few and long."""
    from ... import parallel
    B, L, R = u.shape
    if B < 1 or not (u.is_contiguous() and c.is_contiguous()) or u.dtype != torch.bfloat16:
        return 1
    splits = parallel._auto_local_splits(B, L, chunk_size, 1, u.device)
    if splits > 1 and not C.lib().fracssm_scan_fused_supported(B * splits, L // splits, R, c.shape[-1],
                                                               chunk_size, C.dt(u), C.dt(c)):
        return 1
    return splits


def _launch(u, c, kappa, rho, chunk_size, initial_state, want_final, final_fp32, path_code, check=False):
    B, L, R = u.shape
    M = c.shape[-1]
    final_state_dtype = torch.float32 if final_fp32 else torch.bfloat16
    u, c, kappa, rho = C.rows(u), C.rows(c), C.rows(kappa), C.rows(rho)
    init = None if initial_state is None else initial_state.contiguous()
    h = torch.empty(B, L, R, device=u.device, dtype=u.dtype)
    fin = torch.empty(B, R, M, device=u.device, dtype=final_state_dtype) if want_final else None
    if L == 0:      # no token: the state passes through unchanged (zeros without an initial state)
        if want_final:
            if init is None:
                fin.zero_()
            else:
                fin.copy_(init)
        return h, fin
    if B > 0:
        lib = C.lib()
        with C.trace("frac_scan"), torch.cuda.device(u.device):
            nbytes = lib.fracssm_frac_scan_workspace_bytes(B, max(L, 1), R, M, chunk_size, path_code)
            ws = torch.empty(max(nbytes, 256), device=u.device, dtype=torch.uint8)
            C.check(lib.fracssm_frac_scan_fwd(
                C.ptr(u), C.dt(u), u.stride(0), u.stride(1), C.ptr(c), C.ptr(kappa), C.dt(c),
                c.stride(0), c.stride(1), kappa.stride(0), kappa.stride(1), C.ptr(rho), rho.stride(0),
                rho.stride(1), C.ptr(init), C.ptr(h), C.ptr(fin), C.dt_of(final_state_dtype),
                C.ptr(ws), ws.numel(), B, L, R, M, chunk_size, path_code, C.stream_of(u)), "frac_scan")
            if check and L > 0 and path_code != C.PATH_STAGED and u.is_contiguous() and \
                    lib.fracssm_scan_fused_supported(B, L, R, M, chunk_size, C.dt(u), C.dt(c)):
                C.check(lib.fracssm_scan_fused_status(C.ptr(ws), C.stream_of(u)), "frac_scan")
    if fin is None:
        fin = torch.empty(0, device=u.device, dtype=final_state_dtype)
    return h, fin


# Registered as a torch custom op (with a shape-only "fake" implementation) so that callers can put
# the scan inside torch.compile(fullgraph=True), as the reference does for its ops
# (frac_ssm/ops/triton/chunk_state.py:243-302).  Forward only: asking for gradients raises.
@torch.library.custom_op("frac_ssm_b200::frac_scan_fwd", mutates_args=())
def _frac_scan_fwd_op(u: torch.Tensor, c: torch.Tensor, kappa: torch.Tensor, rho: torch.Tensor,
                      chunk_size: int, initial_state: Optional[torch.Tensor], want_final: bool,
                      final_fp32: bool, path_code: int) -> Tuple[torch.Tensor, torch.Tensor]:
    return _launch(u, c, kappa, rho, chunk_size, initial_state, want_final, final_fp32, path_code)


@_frac_scan_fwd_op.register_fake
def _(u, c, kappa, rho, chunk_size, initial_state, want_final, final_fp32, path_code):
    B, L, R = u.shape
    M = c.shape[-1]
    fdt = torch.float32 if final_fp32 else torch.bfloat16
    fin = torch.empty((B, R, M) if want_final else (0,), device=u.device, dtype=fdt)
    return torch.empty(B, L, R, device=u.device, dtype=u.dtype), fin


def _no_backward(ctx, *grads):
    raise NotImplementedError("frac_ssm_b200 implements the forward pass only")


_frac_scan_fwd_op.register_autograd(_no_backward)


__all__ = ["frac_scan"]
