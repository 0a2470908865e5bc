"""Multi-GPU use of the scan: one process per GPU, `torch.distributed` for the plumbing.

Two ways to shard, both new with respect to the reference (which has no distributed code):

* rows — dim 0 (batch x heads) is split across ranks.  Every stage is independent across dim 0
  (`frac_ssm/ops/triton/chunk_cumsum.py:57` and every other grid starts with the row index), so
  the scan needs no communication: `shard_rows` just gives each rank its slice.
* sequence — each rank owns a contiguous segment of tokens.  A segment acts on the state as
  S -> D (.) S + F with D the product of its decays and F its own contribution from a zero
  state; these pairs compose associatively (the segment summaries of
  `frac_ssm/ops/cute/state_passing.py:144-199`), so one all-gather of (D, F) per rank gives
  every rank its true incoming state, after which it scans its segment once.

The stage functions are taken from an `ops` object so the host logic can be exercised on CPU
ranks (gloo) with CPU stage functions supplied by the tests; the default is the CUDA extension.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_rows(n_rows: int, rank: int, world: int) -> slice:
    """Contiguous, balanced range of dim-0 rows owned by `rank` (earlier ranks get the remainder)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of size {world}")
    base, extra = divmod(n_rows, world)
    lo = rank * base + min(rank, extra)
    return slice(lo, lo + base + (1 if rank < extra else 0))


def shard_tokens(seqlen: int, chunk_size: int, rank: int, world: int) -> slice:
    """Token range of `rank` for sequence sharding: whole chunks, balanced, in rank order."""
    nchunks = (seqlen + chunk_size - 1) // chunk_size
    sl = shard_rows(nchunks, rank, world)
    return slice(sl.start * chunk_size, min(sl.stop * chunk_size, seqlen))


class CudaStageOps:
    """Stage functions on the CUDA extension (the product path)."""

    @staticmethod
    def segment_summary(u, kappa, rho, chunk_size):
        """(log-decay total [B, M], final state from a zero state [B, R, M]) of a segment."""
        from .ops.b200 import stages
        lcr, cd = stages._cumsum(rho, chunk_size, True)
        states = stages.chunk_state(u, kappa, lcr, chunk_size, state_fp32=True)
        _, fin = stages._state_passing(states, cd, None, torch.float32, torch.float32)
        return cd.sum(dim=1), fin

    @staticmethod
    def scan(u, c, kappa, rho, chunk_size, initial_state):
        from .ops.b200.frac_scan import frac_scan
        return frac_scan(u, c, kappa, rho, chunk_size, initial_state, True,
                         final_state_dtype=torch.float32)


def incoming_state(log_decay_all, final_all, rank, initial_state=None):
    """State entering segment `rank`, from the gathered summaries of all segments.

    log_decay_all [G, B, M], final_all [G, B, R, M]; segment g maps S -> exp(D_g) (.) S + F_g.
    """
    G = final_all.shape[0]
    if log_decay_all.shape[0] != G:
        raise ValueError("segment summaries disagree on the number of segments")
    state = torch.zeros_like(final_all[0]) if initial_state is None else initial_state.to(final_all.dtype)
    for g in range(rank):
        state = torch.exp(log_decay_all[g])[:, None, :] * state + final_all[g]
    return state


def seq_parallel_scan(u, c, kappa, rho, chunk_size, initial_state=None, return_final_state=False,
                      group=None, ops=None):
    """Scan a sequence whose tokens are split across the ranks of `group` (in rank order).

    Every rank passes ITS segment (`[B, L_local, ...]`; all segments but the last must be a
    multiple of `chunk_size` long) and the same `initial_state` (the state before token 0 of
    the whole sequence, or None).  Returns this rank's `h` and, if requested, the final state of
    the WHOLE sequence (broadcast from the last rank).
    """
    ops = CudaStageOps if ops is None else ops
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    B, L_local, R = u.shape
    M = c.shape[-1]
    if rank < world - 1 and L_local % chunk_size != 0:
        raise ValueError(
            f"segment of rank {rank} has {L_local} tokens, not a multiple of chunk_size {chunk_size}")
    if world == 1:
        h, fin = ops.scan(u, c, kappa, rho, chunk_size, initial_state)
        return (h, fin) if return_final_state else h

    log_decay, fin0 = ops.segment_summary(u, kappa, rho, chunk_size)
    packed = torch.cat([fin0.reshape(B, R * M), log_decay.reshape(B, M)], dim=1).float().contiguous()
    gathered = torch.empty(world * B, R * M + M, dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(gathered, packed, group=group)   # rank-major concatenation on dim 0
    gathered = gathered.view(world, B, R * M + M)
    final_all = gathered[:, :, : R * M].reshape(world, B, R, M)
    decay_all = gathered[:, :, R * M:]
    init = incoming_state(decay_all, final_all, rank, initial_state)
    h, fin = ops.scan(u, c, kappa, rho, chunk_size, init)
    if not return_final_state:
        return h
    fin = fin.float().contiguous()
    last = dist.get_global_rank(group, world - 1) if group is not None else world - 1
    dist.broadcast(fin, src=last, group=group)
    return h, fin


__all__ = ["shard_rows", "shard_tokens", "CudaStageOps", "incoming_state", "seq_parallel_scan"]
