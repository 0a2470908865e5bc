"""CPU oracle for the FRAC fractional-SSM chunked scan (forward).

TEST INFRASTRUCTURE ONLY.  This file restates, in plain torch on the CPU, the
algorithm of the pure-PyTorch reference of quorbix/frac-ssm-kernels.  It is the
checker the CUDA kernels are compared with, and the CPU arm of the benchmark.
Nothing in the shipped package imports it: the product path is the CUDA
extension and fails loudly when that is missing.

Parity status: PINNED.  `tests/golden/*.pt` hold outputs of the reference's own
`frac_ssm.ops.refs`, `frac_ssm.layers.refs` and `rmsnorm_gated_ref` functions,
produced by `tests/golden/make_golden.py`; `tests/test_oracle_golden.py` checks
every function below against them.

Two precision modes mirror the reference's `upcast` switch:
  exact=True   decay terms in float64, contractions in float32/float64
               (the reference's "truth", `upcast=True`)
  exact=False  working precision: decay in float32, contractions in the input
               dtype (`upcast=False`)

Conventions: dim 0 is the flattened (batch, head) index, T is the chunk length,
N = ceil(L / T) chunks, R the head width, M the number of modes.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

RHO_FLOOR = 1e-6


def _nchunks(L: int, T: int) -> int:
    return (L + T - 1) // T


def _pad_tokens(x: torch.Tensor, Lp: int, mode: str = "zero") -> torch.Tensor:
    """Extend dim 1 of x to Lp tokens, with zeros or by repeating the last row."""
    L = x.shape[1]
    if Lp == L:
        return x
    if mode == "zero":
        return F.pad(x, (0, 0, 0, Lp - L))
    tail = x[:, L - 1 : L, :].expand(-1, Lp - L, -1)
    return torch.cat((x, tail), dim=1)


def log_decay(rho: torch.Tensor, exact: bool = False) -> torch.Tensor:
    """log of the decay with the 1e-6 floor; float32 result.

    Follows frac_ssm/ops/refs/frac_scan.py:31-34.
    """
    if exact:
        return torch.log(rho.double().clamp(min=RHO_FLOOR)).float()
    return torch.log(rho.clamp(min=RHO_FLOOR))


def chunk_cumsum(log_rho: torch.Tensor, T: int, exact: bool = False):
    """Inclusive running sum of log_rho inside each chunk, plus chunk totals.

    Follows frac_ssm/ops/refs/chunk_cumsum.py:19-35: a partial last chunk is
    zero-filled, so its total is the sum over its valid tokens.
    Returns (log_cum_rho [B, L, M], chunk_decay [B, N, M]).
    """
    B, L, M = log_rho.shape
    N = _nchunks(L, T)
    work = log_rho.double() if exact else log_rho.float()
    work = _pad_tokens(work, N * T, "zero").reshape(B, N, T, M)
    run = work.cumsum(dim=2)
    totals = run[:, :, T - 1, :].contiguous()
    lcr = run.reshape(B, N * T, M)[:, :L]
    if exact:
        lcr = lcr.to(log_rho.dtype)
        totals = totals.to(log_rho.dtype)
    return lcr, totals


def chunk_state(u, kappa, lcr, T: int, state_fp32: bool = True, exact: bool = True):
    """Per-chunk state contribution decayed to the end of its chunk.

    states[b, n, r, m] = sum_t u[t, r] * kappa[t, m] * exp(lcr[last, m] - lcr[t, m])
    Follows frac_ssm/ops/refs/chunk_state.py:31-53.  In a partial chunk the
    last valid lcr row is repeated, u and kappa are zero.
    """
    B, L, R = u.shape
    M = kappa.shape[-1]
    N = _nchunks(L, T)
    Lp = N * T
    u4 = _pad_tokens(u, Lp, "zero").reshape(B, N, T, R)
    k4 = _pad_tokens(kappa, Lp, "zero").reshape(B, N, T, M)
    g4 = _pad_tokens(lcr, Lp, "repeat")
    g4 = g4.to(torch.float64 if exact else torch.float32).reshape(B, N, T, M)
    mul_dtype = torch.float32 if exact else u.dtype
    to_end = torch.exp(g4[:, :, T - 1 : T, :] - g4).float()
    weight = (to_end * k4.float()).to(mul_dtype)
    states = torch.einsum("bntr,bntm->bnrm", u4.to(mul_dtype), weight)
    return states.to(torch.float32 if state_fp32 else u.dtype)


def state_passing(states, chunk_decay, initial_state=None, out_dtype=None, exact: bool = False):
    """Carry the state across chunks.

    states_acc[n] is the state BEFORE chunk n; the carry is
    run <- exp(chunk_decay[n]) * run + states[n].
    Follows frac_ssm/ops/refs/state_passing.py:12-31, including its choice of
    accumulating in bfloat16 when `states` is bfloat16 and exact is False.
    Returns (states_acc [B, N, R, M], final_state [B, R, M]).
    """
    B, N, R, M = states.shape
    out_dtype = states.dtype if out_dtype is None else out_dtype
    if exact:
        acc_dtype, exp_dtype = torch.float64, torch.float64
    else:
        acc_dtype = torch.bfloat16 if states.dtype == torch.bfloat16 else torch.float32
        exp_dtype = torch.float32
    if initial_state is None:
        run = torch.zeros(B, R, M, dtype=acc_dtype, device=states.device)
    else:
        run = initial_state.to(acc_dtype)
    before = torch.empty(B, N, R, M, dtype=out_dtype, device=states.device)
    for n in range(N):
        before[:, n] = run.to(out_dtype)
        keep = torch.exp(chunk_decay[:, n].to(exp_dtype)).to(acc_dtype)[:, None, :]
        run = torch.addcmul(states[:, n].to(acc_dtype), keep, run)
    return before, run.to(states.dtype)


def chunk_w(c, kappa, lcr, T: int, exact: bool = False):
    """Causal intra-chunk interaction matrix.

    W[b, n, t, k] = [k <= t] * sum_m c[t, m] * exp(lcr[t, m] - lcr[k, m]) * kappa[k, m]
    Follows frac_ssm/ops/refs/chunk_w.py:12-37 (the difference is masked to
    -inf above the diagonal before the exponential).  float32 result.
    """
    B, L, M = lcr.shape
    N = _nchunks(L, T)
    Lp = N * T
    wd = torch.float64 if exact else torch.float32
    c4 = _pad_tokens(c, Lp, "zero").reshape(B, N, T, M).to(wd)
    k4 = _pad_tokens(kappa, Lp, "zero").reshape(B, N, T, M).to(wd)
    g4 = _pad_tokens(lcr, Lp, "repeat").reshape(B, N, T, M).to(wd)
    gap = g4[:, :, :, None, :] - g4[:, :, None, :, :]  # [B, N, t, k, M]
    idx = torch.arange(T, device=lcr.device)
    above = idx[:, None] < idx[None, :]
    gap = gap.masked_fill(above[..., None], float("-inf"))
    W = (c4[:, :, :, None, :] * torch.exp(gap) * k4[:, :, None, :, :]).sum(dim=-1)
    return W.float()


def chunk_readout(u, c, states_acc, W, lcr, T: int, exact: bool = False):
    """h = (c * exp(lcr)) . states_acc^T  +  W . u   per chunk.

    Follows frac_ssm/ops/refs/chunk_readout.py:15-39; here a partial chunk pads
    lcr with zeros (c is zero there, so the choice is immaterial).
    """
    B, L, R = u.shape
    M = c.shape[-1]
    N = _nchunks(L, T)
    Lp = N * T
    u4 = _pad_tokens(u, Lp, "zero").reshape(B, N, T, R)
    c4 = _pad_tokens(c, Lp, "zero").reshape(B, N, T, M)
    g4 = _pad_tokens(lcr, Lp, "zero").reshape(B, N, T, M)
    mul_dtype = torch.float32 if exact else u.dtype
    since_start = torch.exp(g4.to(torch.float64 if exact else torch.float32)).float()
    read = (c4.float() * since_start).to(mul_dtype)
    carried = torch.einsum("bntm,bnrm->bntr", read, states_acc.to(mul_dtype))
    local = torch.einsum("bntk,bnkr->bntr", W.to(mul_dtype), u4.to(mul_dtype))
    return (carried + local).reshape(B, Lp, R)[:, :L]


def frac_scan(u, c, kappa, rho, T: int, initial_state=None, return_final_state=False,
              exact: bool = False):
    """Composed chunked scan, stage by stage as frac_ssm/ops/refs/frac_scan.py:27-54."""
    assert rho.dtype == torch.float32, "rho must be float32 for numerical stability"
    if initial_state is not None:
        assert initial_state.dtype == torch.float32, "initial_state must be float32"
    lr = log_decay(rho, exact)
    lcr, totals = chunk_cumsum(lr, T, exact)
    fp32_state = exact or u.dtype != torch.bfloat16
    st = chunk_state(u, kappa, lcr, T, state_fp32=fp32_state, exact=exact)
    before, last = state_passing(st, totals, initial_state, exact=exact)
    W = chunk_w(c, kappa, lcr, T, exact)
    h = chunk_readout(u, c, before, W, lcr, T, exact)
    return (h, last) if return_final_state else h


def frac_scan_slabs(u, c, kappa, rho, T: int, initial_state=None, return_final_state=False,
                    exact: bool = False, slab: int = 1):
    """frac_scan evaluated over slices of dim 0 (every stage is independent across dim 0).

    chunk_w materialises [B, N, T, T, M]; slicing bounds that at large shapes.
    """
    hs, fs = [], []
    for lo in range(0, u.shape[0], slab):
        hi = min(lo + slab, u.shape[0])
        init = None if initial_state is None else initial_state[lo:hi]
        h, f = frac_scan(u[lo:hi], c[lo:hi], kappa[lo:hi], rho[lo:hi], T, init, True, exact)
        hs.append(h)
        fs.append(f)
    h = torch.cat(hs, 0)
    return (h, torch.cat(fs, 0)) if return_final_state else h


def token_recurrence(u, c, kappa, rho, initial_state=None):
    """Independent check: the unchunked recurrence in float64.

    S_t = max(rho_t, 1e-6) * S_{t-1} + u_t (x) kappa_t ;  h_t = S_t . c_t
    This is the single-token update of frac_ssm/models/modeling_frac.py:159-179
    written in the scan's [B, R, M] state layout.
    Returns (h [B, L, R] float64, final_state [B, R, M] float64).
    """
    B, L, R = u.shape
    M = c.shape[-1]
    S = torch.zeros(B, R, M, dtype=torch.float64) if initial_state is None else initial_state.double()
    ud, cd, kd = u.double(), c.double(), kappa.double()
    rd = rho.double().clamp(min=RHO_FLOOR)
    h = torch.empty(B, L, R, dtype=torch.float64)
    for t in range(L):
        S = rd[:, t, None, :] * S + ud[:, t, :, None] * kd[:, t, None, :]
        h[:, t] = (S * cd[:, t, None, :]).sum(-1)
    return h, S


# --------------------------------------------------------------------------
# layer-level stages around the scan
# --------------------------------------------------------------------------

def compute_params(dyn, rw, x_conv, attention_mask, dt_bias, read_residual_logit,
                   write_residual_scale, base_log_tau, num_heads, head_dim, num_modes,
                   read_temp, dt_min, dt_max, alpha_min, alpha_max, lambda_min, lambda_max,
                   exact: bool = False):
    """Elementwise parameter prep after the two projections.

    dyn [B, L, 3H] holds (dt, alpha, lambda) logits per head; rw [B, L, 2*H*M]
    holds read then write residual logits.  Follows
    frac_ssm/layers/refs/compute_params.py:36-121 from the point where `dyn` and
    `rw` exist.  Returns head-major (u [BH, L, R], c, kappa, rho [BH, L, M]).
    """
    wd = torch.float64 if exact else torch.float32
    H, R, M = num_heads, head_dim, num_modes
    B, L, _ = x_conv.shape
    dyn = dyn.to(wd)
    dt_l, al_l, la_l = dyn.split(H, dim=-1)
    dt = F.softplus(dt_l + dt_bias.to(wd)).clamp(min=dt_min, max=dt_max)
    alpha = alpha_min + torch.sigmoid(al_l) * (alpha_max - alpha_min)
    lam = lambda_min + torch.sigmoid(la_l) * (lambda_max - lambda_min)

    rw = rw.to(wd).view(B, L, 2, H, M)
    log_tau = base_log_tau.to(wd)[None, None, None, :]
    prior = -alpha[..., None] * log_tau
    read_gate = torch.sigmoid(read_residual_logit.to(wd))
    write_gate = torch.sigmoid(write_residual_scale.to(wd))
    read_w = torch.softmax((prior + read_gate * rw[:, :, 0]) / read_temp, dim=-1)
    write_w = torch.softmax(prior + write_gate * rw[:, :, 1], dim=-1)

    tau = torch.exp(log_tau)
    rate = torch.pow(lam.clamp_min(1e-4), 1.0 / alpha.clamp_min(1e-4))
    rho = torch.exp(-dt[..., None] * (rate[..., None] / tau.clamp_min(1e-6)))
    rho = rho.clamp(min=1e-6, max=1.0 - 1e-6)
    kappa = (1.0 - rho) * write_w

    def head_major(x, width):
        return x.permute(0, 2, 1, 3).reshape(B * H, L, width)

    u = x_conv.view(B, L, H, R)
    if exact:
        u = u.double()
    u_f = head_major(u, R)
    c_f, k_f, r_f = head_major(read_w, M), head_major(kappa, M), head_major(rho, M)
    if attention_mask is not None:
        keep = attention_mask[:, None, :].expand(B, H, L).reshape(B * H, L, 1).to(k_f.dtype)
        k_f = k_f * keep
        r_f = r_f * keep + (1.0 - keep)
    return u_f, c_f, k_f, r_f


def skip_mix(mixed_flat, x_conv, D, num_heads, head_dim, out_dtype=None, exact: bool = False):
    """out[b, l, h*R + r] = mixed_flat[b*H + h, l, r] + x_conv[b, l, h*R + r] * D[h, r].

    Follows frac_ssm/layers/refs/output_mix.py:9-26.
    """
    out_dtype = x_conv.dtype if out_dtype is None else out_dtype
    B, L, _ = x_conv.shape
    H, R = num_heads, head_dim
    if exact:
        mixed_flat, x_conv = mixed_flat.double(), x_conv.double()
    y = mixed_flat.view(B, H, L, R).permute(0, 2, 1, 3)
    y = y + x_conv.view(B, L, H, R).to(y.dtype) * D[None, None].to(y.dtype)
    y = y.reshape(B, L, H * R)
    return y if exact else y.to(out_dtype)


def rmsnorm_gated(x, weight, gate=None, eps: float = 1e-6, exact: bool = False):
    """y = w * rmsnorm(x * silu(gate)) over the last dim.

    Follows frac_ssm/modules/rmsnorm_gated.py:8-24.
    """
    wd = torch.float64 if exact else torch.float32
    y = x.to(wd)
    if gate is not None:
        y = y * F.silu(gate.to(wd))
    y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps)
    if exact:
        return weight.to(wd) * y
    return weight * y.to(x.dtype)


# --------------------------------------------------------------------------
# seeded input generators (CPU generators, so seeds are portable)
# --------------------------------------------------------------------------

_TAU = (1.0, 65536.0)


def uniform_log_rho(B, L, M, seed=0):
    """log of U(0,1) clipped to [0.01, 0.99]; the 'random' generator of tests/utils.py:22-26."""
    g = torch.Generator().manual_seed(seed)
    return torch.rand(B, L, M, generator=g).clamp(0.01, 0.99).log()


def model_like_log_rho(B, L, M, seed=0):
    """Decays shaped like the model's: tests/utils.py:29-44 (smoothed softplus dt,
    alpha in U(0.2,0.95), lambda in U(0.25,4), geometric tau from 1 to 65536)."""
    g = torch.Generator().manual_seed(seed)
    tau = torch.linspace(math.log(_TAU[0]), math.log(_TAU[1]), M).exp()
    raw = torch.randn(B, L, generator=g)
    raw = F.avg_pool1d(raw[:, None, :], 4, stride=1, padding=2)[..., :L].squeeze(1)
    dt = F.softplus(raw).clamp(1e-4, 1.0)
    alpha = 0.20 + 0.75 * torch.rand(B, L, generator=g)
    lam = 0.25 + 3.75 * torch.rand(B, L, generator=g)
    rate = lam ** (1.0 / alpha)
    rho = torch.exp(-dt[..., None] * rate[..., None] / tau).clamp(1e-6, 1.0 - 1e-6)
    return rho.log()


LOG_RHO_GENS = {"random": uniform_log_rho, "model_like": model_like_log_rho}


def scan_inputs(B, L, R, M, dtype=torch.bfloat16, gen="model_like", seed=0, scale=0.25):
    """Scan-level inputs as the reference's tests draw them (tests/test_frac_scan.py:44-58),
    from a CPU generator.  Returns u, c, kappa (dtype), rho, initial_state (float32)."""
    g = torch.Generator().manual_seed(seed)
    u = (scale * torch.randn(B, L, R, generator=g)).to(dtype)
    c = (scale * torch.randn(B, L, M, generator=g)).to(dtype)
    kappa = (scale * torch.randn(B, L, M, generator=g)).to(dtype)
    rho = LOG_RHO_GENS[gen](B, L, M, seed=seed + 1).exp()
    init = scale * torch.randn(B, R, M, generator=g)
    return u, c, kappa, rho, init


def layer_inputs(batch, L, H, R, M, G=1, seed=0, dtype=torch.bfloat16):
    """Layer-level synthetic inputs with the benchmark's stated distributions.

    x, Bt, Ct, z ~ N(0,1) in `dtype`; dt = softplus(N(0,1) - 4); A = -exp(U[0, ln 16]);
    D ~ N(0,1); alpha ~ U(0.3, 0.9) per head (float32).  Mapped through the
    reference's prep math with lam := -A, gates 1, read_temp 1, group g = h // (H/G):
      rho = clamp(exp(-dt * lam^(1/alpha) / tau), 1e-6, 1-1e-6), prior = -alpha * log tau,
      c = softmax_m(prior + Ct), kappa = (1 - rho) * softmax_m(prior + Bt), u = x.
    Returns a dict with scan-level tensors (head-major) and the epilogue tensors.
    """
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(batch, L, H, R, generator=g).to(dtype)
    Bt = torch.randn(batch, L, G, M, generator=g).to(dtype)
    Ct = torch.randn(batch, L, G, M, generator=g).to(dtype)
    z = torch.randn(batch, L, H * R, generator=g).to(dtype)
    dt = F.softplus(torch.randn(batch, L, H, generator=g) - 4.0)
    A = -torch.exp(torch.rand(H, generator=g) * math.log(16.0))
    D = torch.randn(H, generator=g)
    alpha = 0.3 + 0.6 * torch.rand(H, generator=g)
    log_tau = torch.linspace(math.log(_TAU[0]), math.log(_TAU[1]), M)
    rate = (-A) ** (1.0 / alpha)                                   # [H]
    rho = torch.exp(-dt[..., None] * rate[None, None, :, None] / log_tau.exp())
    rho = rho.clamp(1e-6, 1.0 - 1e-6)                              # [b, L, H, M]
    prior = -alpha[:, None] * log_tau[None, :]                     # [H, M]
    grp = torch.arange(H) // (H // G)
    cw = torch.softmax(prior + Ct.float()[:, :, grp], dim=-1)
    ww = torch.softmax(prior + Bt.float()[:, :, grp], dim=-1)
    kap = (1.0 - rho) * ww

    def hm(t, w):
        return t.permute(0, 2, 1, 3).reshape(batch * H, L, w).contiguous()

    return {
        "u": hm(x, R), "c": hm(cw, M).to(dtype), "kappa": hm(kap, M).to(dtype),
        "rho": hm(rho, M).float(), "x_conv": x.reshape(batch, L, H * R), "z": z,
        "D": D[:, None].expand(H, R).contiguous(), "H": H, "R": R, "M": M,
    }
