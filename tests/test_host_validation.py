"""Host-side argument checks mirror the reference's messages (runs on CPU tensors)."""

import pytest
import torch

from frac_ssm_b200 import ops
from frac_ssm_b200.ops.b200 import frac_scan as backend_scan


def test_cu_seqlens_rejected():
    x = torch.zeros(1, 4, 2)
    with pytest.raises(NotImplementedError, match="cu_seqlens is not supported yet"):
        ops.frac_scan(x, x, x, x, 4, cu_seqlens=torch.tensor([0, 4]))


def test_unknown_backend():
    x = torch.zeros(1, 4, 2)
    with pytest.raises(ValueError, match="Unknown backend"):
        ops.frac_scan(x, x, x, x, 4, impl="nope")


def test_rho_and_initial_state_dtype():
    u = torch.zeros(1, 4, 2, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="rho must be float32"):
        backend_scan(u, u, u, u, 4)
    rho = torch.ones(1, 4, 2)
    with pytest.raises(AssertionError, match="initial_state must be float32"):
        backend_scan(u, u, u, rho, 4, torch.zeros(1, 2, 2, dtype=torch.bfloat16))


@pytest.mark.parametrize("fn,args,pattern", [
    (ops.chunk_cumsum, (torch.zeros(4, 2), 4), "3D"),
    (ops.chunk_cumsum, (torch.zeros(1, 4, 2), 4), "CUDA"),
    (ops.chunk_w, (torch.zeros(4, 2), torch.zeros(1, 4, 2), torch.zeros(1, 4, 2), 32), "3D"),
    (ops.chunk_w, (torch.zeros(1, 4, 2),) * 3 + (32,), "CUDA"),
    (ops.state_passing, (torch.zeros(1, 1, 2), torch.zeros(1, 1, 2)), "4D"),
    (ops.chunk_readout, (torch.zeros(4, 2),) * 5 + (4,), "3D"),
    (ops.chunk_fused_readout, (torch.zeros(4, 2),) * 5 + (4,), "3D"),
    (ops.chunk_state, (torch.zeros(1, 4, 2),) * 3 + (4,), "CUDA"),
])
def test_stage_messages(fn, args, pattern):
    with pytest.raises(AssertionError, match=pattern):
        fn(*args)


def test_cute_backend_is_reported_absent():
    ok, why = ops.cute_supported()
    assert not ok and "b200" in why


def test_layer_and_mixer_wrappers_refuse_cpu_tensors():
    """No CPU fallback anywhere: the layer / mixer wrappers refuse host tensors before touching the library."""
    from frac_ssm_b200.layers import scan_epilogue, scan_epilogue_apply, scan_epilogue_sumsq
    from frac_ssm_b200.models.modeling_frac import causal_conv_silu
    h, x = torch.zeros(2, 4, 8), torch.zeros(1, 4, 16)
    D, w = torch.zeros(2, 8), torch.ones(16)
    for call in (lambda: scan_epilogue(h, x, x, D, w, 2, 8),
                 lambda: scan_epilogue_sumsq(h, x, x, D, 2, 8),
                 lambda: scan_epilogue_apply(h, x, x, D, w, 2, 8, torch.zeros(1, 4), 16)):
        with pytest.raises(AssertionError, match="CUDA"):
            call()
    with pytest.raises(AssertionError, match="CUDA"):
        causal_conv_silu(x, torch.zeros(16, 1, 4), None)


def test_shard_heads_covers_every_head_once():
    from frac_ssm_b200 import parallel
    for heads, world in ((64, 8), (24, 5), (3, 4)):
        seen = []
        for r in range(world):
            sl = parallel.shard_heads(heads, r, world)
            seen.extend(range(sl.start, sl.stop))
        assert seen == list(range(heads))


def test_misaligned_pointers_are_refused_before_any_launch():
    """The single-pass kernels use 8- and 16-byte accesses: a pointer off a 16-byte boundary is an
    argument error, not a device fault.  Checked on the host with made-up addresses (nothing runs)."""
    import ctypes
    from frac_ssm_b200 import _cabi as C
    lib = C.lib()
    ok, bad = ctypes.c_void_p(0x10000), ctypes.c_void_p(0x10008)
    for which in range(5):
        ptrs = [bad if i == which else ok for i in range(5)]      # u, c, kappa, rho, h
        rc = lib.fracssm_frac_scan_fwd_noalloc(ptrs[0], ptrs[1], ptrs[2], ptrs[3], None, ptrs[4], None, C.F32,
                                               2, 256, 64, 128, None)
        assert rc == 1 and b"16-byte aligned" in lib.fracssm_last_error()
    ws = ctypes.c_void_p(0x20000)
    need = lib.fracssm_segment_summary_workspace_bytes(2, 64, 128)
    for which in range(3):
        ptrs = [bad if i == which else ok for i in range(3)]      # u, kappa, rho
        rc = lib.fracssm_segment_summary(ptrs[0], ptrs[1], C.BF16, ptrs[2], None, ok, ok, ws, need,
                                         2, 256, 64, 128, None)
        assert rc == 1 and b"16-byte aligned" in lib.fracssm_last_error()


def test_conv_head_width_and_missing_pointers_are_argument_errors():
    """fracssm_causal_conv_silu_heads: a head width that does not divide the channels is refused, and
    fracssm_compute_params may leave out u but nothing else (made-up addresses: nothing runs)."""
    import ctypes
    from frac_ssm_b200 import _cabi as C
    lib = C.lib()
    ok = ctypes.c_void_p(0x10000)
    rc = lib.fracssm_causal_conv_silu_heads(ok, C.BF16, 1536, 1536, None, 0, 0, ok, None, C.BF16, ok, C.BF16,
                                            ok, 100, 1, 16, 1536, 4, None)
    assert rc == 1 and b"head width" in lib.fracssm_last_error()
    rc = lib.fracssm_compute_params(ok, C.BF16, 72, 72, ok, C.BF16, 6144, 6144, None, C.BF16, 0, 0, None, 0, 0,
                                    ok, ok, ok, ok, 1.0, 1e-3, 0.1, 0.3, 0.9, 0.25, 4.0, None, None, ok, C.BF16,
                                    ok, 1, 16, 24, 64, 128, None)
    assert rc == 1 and b"null pointer" in lib.fracssm_last_error()
