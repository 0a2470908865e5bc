"""Sequence and head sharding on real devices: emulated on one GPU, and over NCCL when two are present."""

import os
import socket

import pytest
import torch

from oracle import frac_oracle as O
from tests.helpers import TOL_BF16, TOL_F32, close

pytestmark = pytest.mark.gpu


def test_segment_summaries_compose_on_one_gpu():
    """The CUDA stage functions of the sequence-parallel path, run segment after segment on one
    device: summaries -> incoming states -> per-segment scans must equal one scan of the whole."""
    from frac_ssm_b200 import parallel
    B, L, R, M, T, G = 3, 2048, 64, 128, 256, 4
    u, c, kappa, rho, init = (t.cuda() for t in O.scan_inputs(B, L, R, M, gen="model_like", seed=41))
    ops = parallel.CudaStageOps
    toks = [parallel.shard_tokens(L, T, g, G) for g in range(G)]
    summ = [ops.segment_summary(u[:, t], kappa[:, t], rho[:, t], T) for t in toks]
    D = torch.stack([s[0] for s in summ])
    F = torch.stack([s[1] for s in summ])
    hs = []
    for g, t in enumerate(toks):
        s_in = parallel.incoming_state(D, F, g, init)
        h, fin = ops.scan(u[:, t].contiguous(), c[:, t].contiguous(), kappa[:, t].contiguous(),
                          rho[:, t].contiguous(), T, s_in)
        hs.append(h)
    h_ref, f_ref = O.frac_scan_slabs(u.cpu().float(), c.cpu().float(), kappa.cpu().float(), rho.cpu(), T,
                                     init.cpu(), True, exact=True, slab=1)
    close(torch.cat(hs, 1), h_ref, **TOL_BF16)
    close(fin, f_ref, **TOL_F32)


@pytest.mark.parametrize("kdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,L", [(3, 1000), (24, 4096), (200, 129), (1, 128)])
def test_segment_summary_kernel(kdtype, B, L):
    """The one-pass summary kernel against the oracle: final state from a zero state, decay product."""
    from frac_ssm_b200 import parallel
    u, c, kappa, rho, _ = O.scan_inputs(B, L, 64, 128, gen="model_like", seed=B + L)
    kappa = kappa.to(kdtype)
    decay, fin = parallel.CudaStageOps.segment_summary(u.cuda(), kappa.cuda(), rho.cuda(), 256)
    torch.cuda.synchronize()
    lcr, cd = O.chunk_cumsum(O.log_decay(rho, True), 256, True)
    st = O.chunk_state(u.float(), kappa.float(), lcr, 256, exact=True)
    _, f_ref = O.state_passing(st, cd, None, exact=True)
    close(fin, f_ref, **TOL_F32)
    close(decay, torch.exp(cd.double().sum(1)).float(), **TOL_F32)


def test_grouped_summary_leaves_out_the_last_row_of_every_group():
    from frac_ssm_b200 import parallel
    u, c, kappa, rho, _ = (t.cuda() for t in O.scan_inputs(12, 600, 64, 128, gen="model_like", seed=5))
    decay, fin = parallel.CudaStageOps.segment_summary(u, kappa, rho, 256)
    d4, f4 = parallel.CudaStageOps.segment_summary(u, kappa, rho, 256, skip_last_of=4)
    keep = torch.arange(12, device="cuda") % 4 != 3
    assert torch.equal(d4[keep], decay[keep]) and torch.equal(f4[keep], fin[keep])
    assert not d4[~keep].any() and not f4[~keep].any()
    from frac_ssm_b200 import _cabi as C
    with pytest.raises(C.FracSsmError, match="multiple of the group size"):
        parallel.CudaStageOps.segment_summary(u, kappa, rho, 256, skip_last_of=5)


def test_single_process_default_split_matches_plain_scan():
    """Few rows and a long sequence: one process cuts the sequence into sub-segments by default
    (summary pass, state composition, one scan of all sub-segments as rows)."""
    from frac_ssm_b200 import parallel
    B, L, T = 3, 32768, 256
    assert parallel._auto_local_splits(B, L, T, 1, torch.device("cuda")) == 32
    u, c, kappa, rho, init = (t.cuda() for t in O.scan_inputs(B, L, 64, 128, gen="model_like", seed=77))
    from frac_ssm_b200.ops.b200 import frac_scan
    h_ref, f_ref = frac_scan(u, c, kappa, rho, T, init, True, final_state_dtype=torch.float32, path="fused")
    h, fin = parallel.seq_parallel_scan(u, c, kappa, rho, T, init, True)
    close(h, h_ref.cpu(), **TOL_BF16)
    close(fin, f_ref.cpu(), **TOL_F32)
    # the scan's own "auto" path takes the same route for such a shape
    h_auto, f_auto = frac_scan(u, c, kappa, rho, T, init, True)
    assert f_auto.dtype == torch.bfloat16 and torch.equal(h_auto, h)
    close(f_auto, f_ref.cpu(), rtol=2e-2, atol=2e-2)
    h_only = frac_scan(u, c, kappa, rho, T)
    close(h_only, frac_scan(u, c, kappa, rho, T, path="fused").cpu(), **TOL_BF16)
    # the oracle on one row, token by token in float64
    uc, cc, kc, rc = (t[1:2].cpu() for t in (u, c, kappa, rho))
    h_orc, f_orc = O.frac_scan_slabs(uc.float(), cc.float(), kc.float(), rc, T, init[1:2].cpu(), True,
                                     exact=True, slab=1)
    close(h[1:2], h_orc, **TOL_BF16)
    close(fin[1:2], f_orc, **TOL_F32)


def _nccl_worker(rank, world, port, out):
    import torch.distributed as dist
    from frac_ssm_b200 import parallel
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        B, L, R, M, T = 2, 2048, 64, 128, 256
        u, c, kappa, rho, init = O.scan_inputs(B, L, R, M, gen="model_like", seed=43)
        tok = parallel.shard_tokens(L, T, rank, world)
        dev = lambda x: x[:, tok].contiguous().cuda()
        h, fin = parallel.seq_parallel_scan(dev(u), dev(c), dev(kappa), dev(rho), T, init.cuda(), True)
        h_ref, f_ref = O.frac_scan_slabs(u.float(), c.float(), kappa.float(), rho, T, init, True,
                                         exact=True, slab=1)
        ok = torch.allclose(h.float().cpu(), h_ref[:, tok], rtol=2e-2, atol=2e-2) and \
            torch.allclose(fin.cpu(), f_ref, rtol=1e-3, atol=1e-3)
        out[rank] = int(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_sharding_over_nccl():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_nccl_worker, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {0: 1, 1: 1}


def _nccl_heads_worker(rank, world, port, out):
    import torch.distributed as dist
    from frac_ssm_b200 import parallel
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        batch, L, H, R = 2, 300, 16, 64
        g = torch.Generator().manual_seed(17)
        h = torch.randn(batch * H, L, R, generator=g).bfloat16()
        x = torch.randn(batch, L, H * R, generator=g).bfloat16()
        z = torch.randn(batch, L, H * R, generator=g).bfloat16()
        D = torch.randn(H, R, generator=g)
        w = (1 + 0.1 * torch.randn(H * R, generator=g)).bfloat16()
        ref = O.rmsnorm_gated(O.skip_mix(h, x, D, H, R, exact=True), w, z, 1e-6, exact=True)
        hs = parallel.shard_heads(H, rank, world)
        n, cols = hs.stop - hs.start, slice(hs.start * R, hs.stop * R)
        h_loc = h.view(batch, H, L, R)[:, hs].reshape(batch * n, L, R).cuda()
        y = parallel.head_parallel_epilogue(h_loc, x[..., cols].contiguous().cuda(), z[..., cols].contiguous().cuda(),
                                            D[hs].cuda(), w[cols].cuda(), n, R, H, 1e-6)
        out[rank] = int(torch.allclose(y.float().cpu().double(), ref[..., cols], rtol=2e-2, atol=2e-2))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_head_sharded_epilogue_over_nccl():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_nccl_heads_worker, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {0: 1, 1: 1}
