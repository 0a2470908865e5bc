"""Host logic of the multi-GPU paths on CPU ranks (gloo, world size 2 and 3).

The stage functions are the CPU oracle here: what is under test is the partitioning, the
exchange and the composition of segment summaries, not the kernels.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from frac_ssm_b200 import parallel
from oracle import frac_oracle as O


class OracleStageOps:
    @staticmethod
    def segment_summary(u, kappa, rho, T):
        lcr, cd = O.chunk_cumsum(O.log_decay(rho, True), T, True)
        st = O.chunk_state(u.float(), kappa.float(), lcr, T, exact=True)
        _, fin = O.state_passing(st, cd, None, exact=True)
        return torch.exp(cd.double().sum(1)).float(), fin.float()

    @staticmethod
    def scan(u, c, kappa, rho, T, init):
        return O.frac_scan(u.float(), c.float(), kappa.float(), rho, T, init, True, exact=True)


class OracleEpilogueOps:
    """The two passes of the head-sharded epilogue restated with the CPU oracle's pieces."""

    @staticmethod
    def _gated(h, x_conv, gate, D, H, R, gate_bias):
        mixed = O.skip_mix(h, x_conv, D, H, R, out_dtype=torch.float64, exact=True)
        return mixed * torch.nn.functional.silu(gate.double() + gate_bias)

    @staticmethod
    def sumsq(h, x_conv, gate, D, H, R, gate_bias):
        return OracleEpilogueOps._gated(h, x_conv, gate, D, H, R, gate_bias).pow(2).sum(-1).float()

    @staticmethod
    def apply(h, x_conv, gate, D, weight, H, R, sumsq, norm_width, eps, gate_bias):
        v = OracleEpilogueOps._gated(h, x_conv, gate, D, H, R, gate_bias)
        return (v * torch.rsqrt(sumsq.double() / norm_width + eps)[..., None] * weight.double()).float()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, L, R, M, T = 3, 200, 8, 16, 16
        u, c, kappa, rho, init = O.scan_inputs(B, L, R, M, dtype=torch.float32, gen="model_like", seed=7)
        h_ref, f_ref = O.frac_scan(u, c, kappa, rho, T, init, True, exact=True)
        if mode in ("seq", "seq_split"):
            if mode == "seq_split":      # 256 tokens, 2 ranks x 4 sub-segments of 2 chunks each
                L = 256
                u, c, kappa, rho, init = O.scan_inputs(B, L, R, M, dtype=torch.float32, gen="model_like", seed=8)
                h_ref, f_ref = O.frac_scan(u, c, kappa, rho, T, init, True, exact=True)
            tok = parallel.shard_tokens(L, T, rank, world)
            h, fin = parallel.seq_parallel_scan(u[:, tok], c[:, tok], kappa[:, tok], rho[:, tok], T, init,
                                                True, ops=OracleStageOps,
                                                local_splits=4 if mode == "seq_split" else 1)
            ok = torch.allclose(h, h_ref[:, tok], rtol=1e-4, atol=1e-4) and \
                torch.allclose(fin, f_ref, rtol=1e-4, atol=1e-4)
        elif mode.startswith("ragged"):
            # unequal segments (17 chunks over 2 ranks; or a ragged tail): each rank's own candidate for
            # the sub-segment count differs, the ranks must agree on one before they exchange
            L = int(mode[6:])
            B, T = 2, 256
            u, c, kappa, rho, init = O.scan_inputs(B, L, R, M, dtype=torch.float32, gen="model_like", seed=9)
            h_ref, f_ref = O.frac_scan(u, c, kappa, rho, T, init, True, exact=True)
            tok = parallel.shard_tokens(L, T, rank, world)
            h, fin = parallel.seq_parallel_scan(u[:, tok], c[:, tok], kappa[:, tok], rho[:, tok], T, init,
                                                True, ops=OracleStageOps)          # default local_splits
            ok = torch.allclose(h, h_ref[:, tok], rtol=1e-4, atol=1e-4) and \
                torch.allclose(fin, f_ref, rtol=1e-4, atol=1e-4)
        elif mode == "heads":       # a layer's heads spread over the ranks; the norm spans all heads
            batch, H, Rh, Lh = 2, 6, 8, 40
            g = torch.Generator().manual_seed(11)
            hh = torch.randn(batch * H, Lh, Rh, generator=g)
            x = torch.randn(batch, Lh, H * Rh, generator=g)
            z = torch.randn(batch, Lh, H * Rh, generator=g)
            Dk, wk = torch.randn(H, Rh, generator=g), torch.rand(H * Rh, generator=g) + 0.5
            y_ref = O.rmsnorm_gated(O.skip_mix(hh, x, Dk, H, Rh, exact=True), wk, z, 1e-6, exact=True)
            hs = parallel.shard_heads(H, rank, world)
            cols = slice(hs.start * Rh, hs.stop * Rh)
            nloc = hs.stop - hs.start
            h_loc = hh.view(batch, H, Lh, Rh)[:, hs].reshape(batch * nloc, Lh, Rh)
            y = parallel.head_parallel_epilogue(h_loc, x[..., cols].contiguous(), z[..., cols].contiguous(),
                                                Dk[hs], wk[cols], nloc, Rh, H, 1e-6, 0.0,
                                                ops=OracleEpilogueOps)
            ok = torch.allclose(y.double(), y_ref[..., cols], rtol=1e-5, atol=1e-5)
        elif mode == "local":
            # inside an initialised group, process_local=True cuts THIS process's whole sequence and
            # takes part in no exchange (only rank 1 calls it: a collective would hang and time out)
            ok = True
            if rank == 1:
                L = 256
                u, c, kappa, rho, init = O.scan_inputs(B, L, R, M, dtype=torch.float32, gen="model_like", seed=8)
                h_ref, f_ref = O.frac_scan(u, c, kappa, rho, T, init, True, exact=True)
                h, fin = parallel.seq_parallel_scan(u, c, kappa, rho, T, init, True, ops=OracleStageOps,
                                                    local_splits=4, process_local=True)
                ok = torch.allclose(h, h_ref, rtol=1e-4, atol=1e-4) and \
                    torch.allclose(fin, f_ref, rtol=1e-4, atol=1e-4)
        elif mode == "rows":
            rows = parallel.shard_rows(B, rank, world)
            h, fin = OracleStageOps.scan(u[rows], c[rows], kappa[rows], rho[rows], T, init[rows])
            ok = torch.allclose(h, h_ref[rows], rtol=1e-5, atol=1e-5) and \
                torch.allclose(fin, f_ref[rows], rtol=1e-5, atol=1e-5)
        else:  # a segment that is not chunk-aligned must be refused on the offending rank
            ok = True
            if rank < world - 1:      # (the last rank may hold a ragged tail, so it is not called here)
                try:
                    parallel.seq_parallel_scan(u[:, :17], c[:, :17], kappa[:, :17], rho[:, :17], T, None,
                                               False, ops=OracleStageOps)
                    ok = False
                except ValueError:
                    ok = True
        flag = torch.tensor([1 if ok else 0])
        if mode != "misaligned":
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        out[rank] = int(flag.item())
    finally:
        dist.destroy_process_group()


def _run(world, mode):
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, mode, out), nprocs=world, join=True)
        assert dict(out) == {r: 1 for r in range(world)}


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_sharding_matches_single_scan(world):
    _run(world, "seq")


def test_sequence_sharding_with_local_sub_segments():
    _run(2, "seq_split")


@pytest.mark.parametrize("L", [3996, 4352])
def test_sequence_sharding_with_unequal_segments_and_default_splits(L):
    _run(2, f"ragged{L}")


def test_row_sharding_matches_single_scan():
    _run(2, "rows")


def test_process_local_split_ignores_the_group():
    _run(2, "local")


@pytest.mark.parametrize("world", [2, 3])
def test_head_sharded_epilogue_matches_full_norm(world):
    _run(world, "heads")


def test_misaligned_segment_is_refused():
    _run(2, "misaligned")


def test_shard_helpers():
    assert [parallel.shard_rows(10, r, 3) for r in range(3)] == [slice(0, 4), slice(4, 7), slice(7, 10)]
    assert parallel.shard_rows(2, 3, 4) == slice(2, 2)
    toks = [parallel.shard_tokens(1000, 256, r, 2) for r in range(2)]
    assert toks == [slice(0, 512), slice(512, 1000)]
    with pytest.raises(ValueError):
        parallel.shard_rows(4, 4, 4)


def test_single_rank_split_policy():
    """One rank cuts only few-row, long sequences (the extra read must pay for itself); no exchange,
    no host synchronisation."""
    f = lambda B, L: parallel._auto_local_splits(B, L, 256, 1, torch.device("cpu"))
    assert f(24, 1048576) == 8          # 24 rows -> 192 chains
    assert f(29, 1048576) == 1          # enough rows: the plain scan is within reach of the split one
    assert f(24, 16384) == 1            # too short to pay for two more launches
    assert f(3, 32768) == 32            # sub-segments of at least 1024 tokens
    assert f(3, 32768 + 256) == 1       # 129 chunks cannot be halved


def test_incoming_state_composition():
    g = torch.Generator().manual_seed(0)
    D = torch.rand(3, 2, 4, generator=g)
    F = torch.randn(3, 2, 5, 4, generator=g)
    s0 = torch.randn(2, 5, 4, generator=g)
    s = s0.clone()
    for r in range(3):
        torch.testing.assert_close(parallel.incoming_state(D, F, r, s0), s)
        s = D[r][:, None, :] * s + F[r]
    with pytest.raises(ValueError):
        parallel.incoming_state(D[:2], F, 1)


def _leaver_worker(rank, world, port, out):
    """Rank 1 leaves between steps (no collective of its own in flight); rank 0's next exchange must
    end with an error within the process group's short time-out, not hang."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    B, L, R, M, T = 2, 64, 8, 16, 16
    u, c, kappa, rho, init = O.scan_inputs(B, L, R, M, dtype=torch.float32, gen="model_like", seed=21)
    tok = parallel.shard_tokens(L, T, rank, world)
    args = (u[:, tok], c[:, tok], kappa[:, tok], rho[:, tok], T, init, True)
    parallel.seq_parallel_scan(*args, ops=OracleStageOps)          # step 1: everybody is there
    dist.barrier()
    if rank == 1:
        out[rank] = 1
        os._exit(0)                                                  # leaves without a word
    try:
        parallel.seq_parallel_scan(*args, ops=OracleStageOps)      # step 2: the peer is gone
        out[rank] = 0
    except Exception:                                                # noqa: BLE001 - any error is the point
        out[rank] = 1
    os._exit(0)


def test_a_rank_that_leaves_ends_the_others_exchange_with_an_error():
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        ctx = mp.spawn(_leaver_worker, args=(2, port, out), nprocs=2, join=False)
        import time
        t0 = time.time()
        while not ctx.join(timeout=1.0):
            assert time.time() - t0 < 120, "the remaining rank hung instead of failing"
        assert dict(out) == {0: 1, 1: 1}
