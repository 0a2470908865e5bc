"""Multi-GPU use of the scan: one process per GPU, `torch.distributed` for the plumbing.

Three ways to shard, all new with respect to the reference (which has no distributed code):

* rows — dim 0 (batch x heads) is split across ranks.  Every stage is independent across dim 0
  (`frac_ssm/ops/triton/chunk_cumsum.py:57` and every other grid starts with the row index), so
  the scan needs no communication: `shard_rows` just gives each rank its slice.
* sequence — each rank owns a contiguous segment of tokens.  A segment acts on the state as
  S -> D (.) S + F with D the product of its decays and F its own contribution from a zero
  state; these pairs compose associatively (the segment summaries of
  `frac_ssm/ops/cute/state_passing.py:144-199`), so one all-gather of (D, F) per rank gives
  every rank its true incoming state, after which it scans its segment once.

* heads of a whole layer — like rows for the scan itself, but the gated RMSNorm that follows spans
  all heads of a (batch, token) row (`frac_ssm/modules/rmsnorm_gated.py:8-24`): each rank computes
  the sum of squares over its own heads, one all-reduce of a [batch, L] float32 vector adds them,
  and each rank normalises its own columns (`head_parallel_epilogue`).

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
    def segment_summary(u, kappa, rho, chunk_size, skip_last_of=1):
        """(decay product [B, M], final state from a zero state [B, R, M]) of a segment, float32.

        One kernel that reads u, kappa and rho once when the shape is covered (R = 64, M = 128,
        bfloat16 u, dense); otherwise the staged kernels (cumsum -> chunk_state -> state_passing).
        `skip_last_of = S > 1`: the rows are groups of S sub-segments of one sequence each and nobody
        needs the summary of a group's last row; the one-kernel path then leaves those rows out
        (their entries are zero), the staged path computes them anyway.
        """
        from . import _cabi as C
        B, L, R = u.shape
        M = kappa.shape[-1]
        if (R == 64 and M == 128 and u.dtype == torch.bfloat16 and L > 0 and B > 0
                and kappa.dtype in (torch.bfloat16, torch.float32)):
            u, kappa, rho = u.contiguous(), kappa.contiguous(), rho.contiguous()
            grouped = skip_last_of > 1
            alloc = torch.zeros if grouped else torch.empty
            fin = alloc(B, R, M, device=u.device, dtype=torch.float32)
            decay = alloc(B, M, device=u.device, dtype=torch.float32)
            lib = C.lib()
            with torch.cuda.device(u.device):
                ws = torch.empty(lib.fracssm_segment_summary_workspace_bytes(B, R, M), device=u.device,
                                 dtype=torch.uint8)
                if grouped:
                    C.check(lib.fracssm_segment_summary_grouped(
                        C.ptr(u), C.ptr(kappa), C.dt(kappa), C.ptr(rho), C.ptr(fin), C.ptr(decay),
                        C.ptr(ws), ws.numel(), B, L, R, M, skip_last_of, C.stream_of(u)), "segment_summary")
                else:
                    C.check(lib.fracssm_segment_summary(
                        C.ptr(u), C.ptr(kappa), C.dt(kappa), C.ptr(rho), None, C.ptr(fin), C.ptr(decay),
                        C.ptr(ws), ws.numel(), B, L, R, M, C.stream_of(u)), "segment_summary")
            return decay, fin
        from .ops.b200 import stages
        lcr, cd = stages._cumsum(rho, chunk_size, True)
        states = stages.chunk_state(u, kappa, lcr, chunk_size, state_fp32=True)
        _, fin = stages._state_passing(states, cd, None, torch.float32, torch.float32)
        return torch.exp(cd.sum(dim=1)), fin

    @staticmethod
    def scan(u, c, kappa, rho, chunk_size, initial_state):
        from .ops.b200.frac_scan import frac_scan
        return frac_scan(u, c, kappa, rho, chunk_size, initial_state, True,
                         final_state_dtype=torch.float32)


def incoming_state(decay_all, final_all, rank, initial_state=None):
    """State entering segment `rank`, from the gathered summaries of all segments.

    decay_all [G, B, M], final_all [G, B, R, M]; segment g maps S -> decay_g (.) S + final_g.
    """
    G = final_all.shape[0]
    if decay_all.shape[0] != G:
        raise ValueError("segment summaries disagree on the number of segments")
    state = torch.zeros_like(final_all[0]) if initial_state is None else initial_state.to(final_all.dtype)
    for g in range(rank):
        state = decay_all[g][:, None, :] * state + final_all[g]
    return state


def _auto_local_splits(B, L_local, chunk_size, world, device, group=None):
    """How many sub-segments every rank cuts its segment into (the same number on all ranks).

    The scan kernels hand the state from tile to tile of a row, so few rows mean few independent
    chains; sub-segments are extra rows.  Splitting costs one more read of u, kappa and rho, so a
    single rank splits only where the chains are what limits the plain scan by a wide margin: at most
    28 rows (one tile step of a chain takes about 2.8 us, a CTA needs about 7.6 us per tile, so
    148 SMs are busy from some 54 rows on, and the extra read costs about 60 % of a scan) and at
    least 32768 tokens (measured on 24 rows x 1,048,576 tokens: 22.7 ms plain, 16.9 ms cut in 8).
    Each rank can only judge its own segment (segments differ by a chunk
    when the chunk count does not divide by the world size, and the last one may be ragged), so the
    ranks agree on the smallest of their candidates with one MIN all-reduce of a single integer;
    candidates are powers of two and a segment that can be cut into S whole-chunk pieces can also be
    cut into any smaller power of two.  Reading the agreed value synchronises the host with the
    device; callers that must not synchronise pass `local_splits` themselves.
    """
    if world == 1 and (B > 28 or L_local < 32768):
        return 1
    s = 1
    while B * s < 148 and L_local % (2 * s * chunk_size) == 0 and L_local // (2 * s) >= 1024:
        s *= 2
    if world == 1:
        return s
    agreed = torch.tensor([s], dtype=torch.int64, device=device)
    dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
    return int(agreed.item())


def seq_parallel_scan(u, c, kappa, rho, chunk_size, initial_state=None, return_final_state=False,
                      group=None, ops=None, local_splits=None, process_local=False):
    """Scan a sequence whose tokens are split across the ranks of `group` (in rank order).

    Every rank passes ITS segment (`[B, L_local, ...]`; all segments but the last must be a
    multiple of `chunk_size` long) and the same `initial_state` (the state before token 0 of
    the whole sequence, or None).  Returns this rank's `h` and, if requested, the final state of
    the WHOLE sequence (broadcast from the last rank).

    `local_splits` (a divisor of L_local / chunk_size, the SAME on every rank) cuts each rank's
    segment into that many sub-segments which are scanned as extra rows: with few (batch x head)
    rows this is what keeps all SMs busy.  By default the ranks agree on a value among themselves
    (one small all-reduce and a host synchronisation, see `_auto_local_splits`).

    `process_local=True` ignores the process group: the tensors are the whole sequence and only the
    sub-segment composition runs (what `frac_scan` does by itself for few rows and many tokens).
    """
    ops = CudaStageOps if ops is None else ops
    if not process_local and dist.is_available() and dist.is_initialized():
        world, rank = dist.get_world_size(group), dist.get_rank(group)
    else:                       # a single process: the same composition without any exchange
        world, rank = 1, 0
    B, L_local, R = u.shape
    M = c.shape[-1]
    if rank < world - 1 and L_local % chunk_size != 0:
        raise ValueError(
            f"segment of rank {rank} has {L_local} tokens, not a multiple of chunk_size {chunk_size}")
    S = (_auto_local_splits(B, L_local, chunk_size, world, u.device, group) if local_splits is None
         else int(local_splits))
    if S < 1 or L_local % S != 0 or (S > 1 and (L_local // S) % chunk_size != 0):
        raise ValueError(f"local_splits={S} does not cut {L_local} tokens into whole chunks")
    if world == 1 and S == 1:
        h, fin = ops.scan(u, c, kappa, rho, chunk_size, initial_state)
        return (h, fin) if return_final_state else h

    Ls = L_local // S
    rows = lambda t: t.contiguous().view(B * S, Ls, t.shape[-1])   # (b, s) becomes the row index
    u_r, c_r, k_r, rho_r = rows(u), rows(c), rows(kappa), rows(rho)
    if rank == world - 1 and ops is CudaStageOps:
        # nobody reads the summary of the whole sequence's last sub-segment(s): the last rank leaves out
        # the last sub-segment of each of its rows
        decay, fin0 = ops.segment_summary(u_r, k_r, rho_r, chunk_size, skip_last_of=S)
    else:
        decay, fin0 = ops.segment_summary(u_r, k_r, rho_r, chunk_size)
    packed = torch.cat([fin0.reshape(B, S, R * M), decay.reshape(B, S, M)], dim=2).float().contiguous()
    if world > 1:
        gathered = torch.empty(world * B, S, R * M + M, dtype=packed.dtype, device=packed.device)
        dist.all_gather_into_tensor(gathered, packed, group=group)   # rank-major concatenation on dim 0
        gathered = gathered.view(world, B, S, R * M + M)
    else:
        gathered = packed[None]
    # virtual segments in sequence order: (rank 0, sub 0), (rank 0, sub 1), ... ; walk them once and
    # keep the states entering this rank's sub-segments
    state = (torch.zeros(B, R, M, dtype=torch.float32, device=u.device) if initial_state is None
             else initial_state.float().clone())
    mine = torch.empty(B, S, R, M, dtype=torch.float32, device=u.device)
    for g in range(rank + 1):
        for sub in range(S):
            if g == rank:
                mine[:, sub] = state
                if sub == S - 1:
                    break
            seg_fin = gathered[g, :, sub, : R * M].reshape(B, R, M)
            seg_dec = gathered[g, :, sub, R * M:]
            state = torch.addcmul(seg_fin, seg_dec[:, None, :], state)
    h, fin = ops.scan(u_r, c_r, k_r, rho_r, chunk_size, mine.view(B * S, R, M))
    h = h.view(B, L_local, R)
    if not return_final_state:
        return h
    fin = fin.view(B, S, R, M)[:, S - 1].float().contiguous()
    if world > 1:
        last = dist.get_global_rank(group, world - 1) if group is not None else world - 1
        dist.broadcast(fin, src=last, group=group)
    return h, fin


__all__ = ["shard_rows", "shard_tokens", "CudaStageOps", "incoming_state", "seq_parallel_scan"]


def shard_heads(num_heads: int, rank: int, world: int) -> slice:
    """Heads owned by `rank` when a layer's heads are spread over `world` ranks."""
    return shard_rows(num_heads, rank, world)


class CudaEpilogueOps:
    """The two passes of the head-sharded epilogue on the CUDA extension."""

    @staticmethod
    def sumsq(h, x_conv, gate, D, num_heads, head_dim, gate_bias):
        from .layers.output_mix import scan_epilogue_sumsq
        return scan_epilogue_sumsq(h, x_conv, gate, D, num_heads, head_dim, gate_bias)

    @staticmethod
    def apply(h, x_conv, gate, D, weight, num_heads, head_dim, sumsq, norm_width, eps, gate_bias):
        from .layers.output_mix import scan_epilogue_apply
        return scan_epilogue_apply(h, x_conv, gate, D, weight, num_heads, head_dim, sumsq, norm_width,
                                   eps, gate_bias)


def head_parallel_epilogue(h, x_conv, gate, D, weight, local_heads, head_dim, total_heads, eps=1e-6,
                           gate_bias=0.0, group=None, ops=CudaEpilogueOps):
    """Skip-mix + gated RMSNorm of a layer whose heads are spread over the ranks of `group`.

    Every rank passes the slices for its own `local_heads` heads: h [batch*local_heads, L, R] (the
    scan's output for those heads), x_conv / gate [batch, L, local_heads*R], D [local_heads, R],
    weight [local_heads*R].  Returns the rank's own columns of the normalised output,
    [batch, L, local_heads*R].  One all-reduce of batch*L float32 values is the only communication.
    """
    sumsq = ops.sumsq(h, x_conv, gate, D, local_heads, head_dim, gate_bias)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(sumsq, op=dist.ReduceOp.SUM, group=group)
    return ops.apply(h, x_conv, gate, D, weight, local_heads, head_dim, sumsq, total_heads * head_dim,
                     eps, gate_bias)


def head_parallel_layer(u, c, kappa, rho, gate, D, weight, local_heads, total_heads, eps=1e-6, gate_bias=0.0,
                        group=None):
    """Scan + skip-mix + gated RMSNorm of a layer whose heads are spread over the ranks of `group`, with
    the epilogue fused into the scan's output stage.  Every rank passes the tensors of its own heads
    (u, c, kappa, rho [batch*local_heads, L, .], gate [batch, L, local_heads*64], D [local_heads, 64],
    weight [local_heads*64]); the only communication is one all-reduce of batch*L float32 sums."""
    from .layers.output_mix import scan_layer_gated, scan_layer_norm, scan_layer_sumsq
    gated, ss, _ = scan_layer_gated(u, c, kappa, rho, gate, D, local_heads, gate_bias)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        sumsq = scan_layer_sumsq(ss)
        dist.all_reduce(sumsq, op=dist.ReduceOp.SUM, group=group)
        return scan_layer_norm(gated, ss, weight, u.shape[-1], eps, sumsq=sumsq,
                               norm_width=total_heads * u.shape[-1])
    return scan_layer_norm(gated, ss, weight, u.shape[-1], eps)
