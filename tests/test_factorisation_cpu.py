"""The single-pass kernel's reformulation of the scan, restated on the CPU and checked against the
oracle: W assembled from an 8x8 base (reference point in the middle of the block) and the sibling
levels 8 / 16 / 32 / 64 (reference point on the boundary between the halves), every factor bounded,
operands rounded to bfloat16, Chat / Khat / the carried state split into bf16 high + low parts.
This guards the MATH the CUDA kernel implements (csrc/scan_fused.cu); the kernel itself is tested on
the GPU."""

import torch

from oracle import frac_oracle as O


def bf(x):
    return x.to(torch.bfloat16).float()


def tile(u, c, kappa, rho, S):
    """One 128-token tile: u [128, R], c / kappa / rho [128, M], incoming state S [M, R] -> h, S_next."""
    M = rho.shape[1]
    g = rho.clamp(min=1e-6).view(16, 2, 4, M)                  # 16 segments of 8 = 2 groups of 4 tokens
    p4 = torch.cumprod(g, dim=2)                               # inclusive prefix inside a group of 4
    s4 = torch.ones_like(g)                                    # product of the tokens after t in its group
    for i in (2, 1, 0):
        s4[:, :, i] = s4[:, :, i + 1] * g[:, :, i + 1]
    G4 = p4[:, :, 3]
    G8 = G4[:, 0] * G4[:, 1]                                   # decay of each 8-token segment
    pre8, suf8 = p4.clone(), s4.clone()
    pre8[:, 1] *= G4[:, 0:1]                                   # prefix from the segment start
    suf8[:, 0] *= G4[:, 1:2]                                   # suffix to the segment end
    cf, kf = c.float().view(16, 8, M), kappa.float().view(16, 8, M)
    cp, ks = cf * pre8.view(16, 8, M), kf * suf8.view(16, 8, M)
    p4v, s4v = p4.view(16, 8, M), s4.view(16, 8, M)
    A0, B0 = torch.empty(16, 8, M), torch.empty(16, 8, M)      # base: reference between tokens 3 and 4
    A0[:, 4:], B0[:, 4:] = cf[:, 4:] * p4v[:, 4:], kf[:, 4:] / p4v[:, 4:]
    A0[:, :4], B0[:, :4] = cf[:, :4] / s4v[:, :4], kf[:, :4] * s4v[:, :4]
    assert B0.abs().max() <= kf.abs().max() * 1.01e24 and A0.abs().max() <= cf.abs().max() * 1.01e18
    t = torch.arange(128)
    W = torch.where(((t[:, None] // 8) == (t[None, :] // 8)) & (t[:, None] >= t[None, :]),
                    bf(A0.view(128, M)) @ bf(B0.view(128, M)).t(), torch.zeros(128, 128))
    for h in (1, 2, 4, 8):                                     # segments per half of a 2s-token block
        X = torch.empty(16, 8, M)
        for w in range(16):
            first = w - (w % h)
            if (w // h) % 2 == 1:                              # second half: A role, back to the boundary
                sig = torch.ones(M)
                for wp in range(first, w):
                    sig = sig * G8[wp]
                X[w] = cp[w] * sig
            else:                                              # first half: B role, forward to the boundary
                sig = torch.ones(M)
                for wp in range(w + 1, first + h):
                    sig = sig * G8[wp]
                X[w] = ks[w] * sig
        assert X.abs().max() <= max(cf.abs().max(), kf.abs().max())         # both factors are <= 1
        X = bf(X.view(128, M))
        s = 8 * h
        owner = ((t[:, None] // (2 * s)) == (t[None, :] // (2 * s))) & \
                ((t[:, None] // s) % 2 == 1) & ((t[None, :] // s) % 2 == 0)
        W = torch.where(owner, X @ X.t(), W)
    E, F = torch.ones(16, M), torch.ones(16, M)                # to the tile's start / end
    for w in range(1, 16):
        E[w] = E[w - 1] * G8[w - 1]
    for w in range(14, -1, -1):
        F[w] = F[w + 1] * G8[w + 1]
    chat, khat = (cp * E[:, None]).view(128, M), (ks * F[:, None]).view(128, M)
    ch, kh, sh = bf(chat), bf(khat), bf(S)
    cl, kl, sl = bf(chat - ch), bf(khat - kh), bf(S - sh)
    uf = u.float()
    h_out = ch @ sh + cl @ sh + ch @ sl + bf(W) @ uf           # low x low dropped, as in the kernel
    S_next = (E[15] * G8[15])[:, None] * S + kh.t() @ uf + kl.t() @ uf
    return h_out, S_next


def emulate(u, c, kappa, rho, init):
    B, L, R = u.shape
    M = c.shape[-1]
    hs, fin = torch.empty(B, L, R), torch.empty(B, R, M)
    for b in range(B):
        S = torch.zeros(M, R) if init is None else init[b].t().contiguous().clone()
        for t0 in range(0, L, 128):
            n = min(128, L - t0)

            def pad(x, val):
                out = torch.full((128, x.shape[-1]), val, dtype=x.dtype)
                out[:n] = x[b, t0:t0 + n]
                return out

            h, S = tile(pad(u, 0.0), pad(c, 0.0), pad(kappa, 0.0), pad(rho, 1.0), S)
            hs[b, t0:t0 + n] = h[:n]
        fin[b] = S.t()
    return hs, fin


def _check(u, c, kappa, rho, init):
    h, fin = emulate(u, c, kappa, rho, init)
    h_ref, f_ref = O.frac_scan_slabs(u.float(), c.float(), kappa.float(), rho, 64, init, True, exact=True)
    assert torch.isfinite(h).all() and torch.isfinite(fin).all()
    torch.testing.assert_close(h.to(torch.bfloat16).float(), h_ref.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(fin, f_ref.float(), rtol=1e-3, atol=1e-3)


def test_factorisation_matches_oracle_on_model_like_and_random_decay():
    for gen, L, seed in (("model_like", 300, 0), ("random", 257, 1)):
        u, c, kappa, rho, init = O.scan_inputs(1, L, 64, 128, dtype=torch.bfloat16, gen=gen, seed=seed)
        _check(u, c, kappa, rho, init)


def test_factorisation_survives_decay_at_the_floor():
    u, c, kappa, rho, _ = O.scan_inputs(1, 256, 64, 128, dtype=torch.bfloat16, gen="random", seed=5)
    rho[:, :, :64] = 1e-7          # below the floor for the whole sequence: factors of 1e-6 per token
    rho[:, 40:200, 64:96] = 1.0    # and spans with no decay at all
    _check(u, c, kappa, rho, None)
