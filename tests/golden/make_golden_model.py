"""Generates tests/golden/model_*.pt: inputs, weights and outputs of the REFERENCE model
(`frac_ssm.models.modeling_frac.FracForCausalLM`) run on CPU in float32.

The reference model calls Triton kernels, which need a GPU.  For this script the names it calls are
pointed at the reference's own pure-PyTorch counterparts (`frac_ssm.layers.refs.*`,
`frac_ssm.ops.refs.frac_scan.frac_scan_ref`, `rmsnorm_ref`, `rmsnorm_gated_ref`, working precision),
so what is recorded is the reference's model code driving the reference's own reference functions.

    python tests/golden/make_golden_model.py --reference /path/to/reference/checkout
"""

from __future__ import annotations

import argparse
import os
import sys

import torch


def build(mf, cfg_kwargs, seed):
    from frac_ssm.models.configuration_frac import FracConfig
    torch.manual_seed(seed)
    cfg = FracConfig(**cfg_kwargs)
    model = mf.FracForCausalLM(cfg).float().eval()
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():   # parameters that start at zero / one get values that matter
        for layer in model.model.layers:
            m = layer.mixer
            m.D.copy_(0.5 * torch.randn(m.D.shape, generator=g))
            m.dt_bias.copy_(0.5 * torch.randn(m.dt_bias.shape, generator=g))
            m.dyn_proj.bias.copy_(0.3 * torch.randn(m.dyn_proj.bias.shape, generator=g))
            m.conv1d.weight.copy_(0.4 * torch.randn(m.conv1d.weight.shape, generator=g))
            if m.conv1d.bias is not None:
                m.conv1d.bias.copy_(0.1 * torch.randn(m.conv1d.bias.shape, generator=g))
            m.out_norm.weight.copy_(1 + 0.1 * torch.randn(m.out_norm.weight.shape, generator=g))
            layer.norm.weight.copy_(1 + 0.1 * torch.randn(layer.norm.weight.shape, generator=g))
            for lin in (m.in_proj, m.rw_proj, m.out_proj, m.dyn_proj):
                lin.weight.copy_(torch.randn(lin.weight.shape, generator=g) / lin.weight.shape[1] ** 0.5)
        model.model.embed_tokens.weight.copy_(torch.randn(model.model.embed_tokens.weight.shape, generator=g))
    return cfg, model


def case(mf, name, cfg_kwargs, batch, L, decode_tokens, masked, seed, out_dir):
    cfg, model = build(mf, cfg_kwargs, seed)
    g = torch.Generator().manual_seed(seed + 2)
    ids = torch.randint(3, cfg.vocab_size, (batch, L + decode_tokens), generator=g)
    mask = None
    if masked:   # left padding on the second sequence
        mask = torch.ones(batch, L, dtype=torch.long)
        mask[1, : L // 4] = 0
    with torch.no_grad():
        out = model(input_ids=ids[:, :L], attention_mask=mask, use_cache=True)
        rec = {"logits": out.logits.clone(),
               "state0": out.past_key_values[0][0].clone(), "conv_state0": out.past_key_values[0][1].clone()}
        past, steps = out.past_key_values, []
        for t in range(decode_tokens):
            o = model(input_ids=ids[:, L + t:L + t + 1], past_key_values=past, use_cache=True)
            past = o.past_key_values
            steps.append(o.logits.clone())
        rec["decode_logits"] = torch.cat(steps, 1) if steps else None
        rec["state_after_decode"] = past[0][0].clone()
        nocache = model(input_ids=ids[:, :L], attention_mask=mask, use_cache=False)
        rec["logits_nocache"] = nocache.logits.clone()
    rec.update(config=cfg_kwargs, input_ids=ids, attention_mask=mask, prefill_len=L,
               state_dict={k: v.clone() for k, v in model.state_dict().items()})
    torch.save(rec, os.path.join(out_dir, name + ".pt"))
    print(name, "logits", tuple(rec["logits"].shape), "max|logit| %.3f" % rec["logits"].abs().max().item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    import frac_ssm.models.modeling_frac as mf
    from frac_ssm.layers.refs import frac_compute_scan_params_ref, frac_skip_mix_ref
    from frac_ssm.modules.rmsnorm import rmsnorm_ref
    from frac_ssm.modules.rmsnorm_gated import rmsnorm_gated_ref
    from frac_ssm.ops.refs.frac_scan import frac_scan_ref

    mf.frac_compute_scan_params = lambda model, x_conv, x, mask=None: frac_compute_scan_params_ref(
        model, x_conv, x, mask, upcast=False)
    mf.frac_skip_mix = lambda model, mixed, x_conv, out_dtype=None: frac_skip_mix_ref(
        model, mixed, x_conv, out_dtype, upcast=False)
    mf.frac_scan = lambda u, c, kappa, rho, T, init=None, ret=False, cu_seqlens=None, impl=None: frac_scan_ref(
        u, c, kappa, rho, T, init, ret, upcast=False)
    mf.RMSNorm.forward = lambda self, x: rmsnorm_ref(x, self.weight, self.variance_epsilon)
    mf.RMSNormGated.forward = lambda self, x, gate=None: rmsnorm_gated_ref(x, self.weight, gate, self.variance_epsilon)

    out_dir = os.path.dirname(os.path.abspath(__file__))
    tiny = dict(vocab_size=61, hidden_size=32, num_hidden_layers=2, num_attention_heads=2, frac_num_modes=16,
                frac_chunk_size=16, frac_gate_bias_init=0.3, tie_word_embeddings=True)
    case(mf, "model_tiny", tiny, batch=2, L=45, decode_tokens=3, masked=False, seed=0, out_dir=out_dir)
    case(mf, "model_tiny_masked", tiny, batch=2, L=40, decode_tokens=2, masked=True, seed=3, out_dir=out_dir)
    wide = dict(vocab_size=53, hidden_size=64, num_hidden_layers=1, num_attention_heads=2, frac_num_modes=128,
                frac_chunk_size=256, tie_word_embeddings=True)       # head_dim 64, 128 modes: the single-pass shape
    case(mf, "model_wide", wide, batch=2, L=300, decode_tokens=2, masked=False, seed=5, out_dir=out_dir)


if __name__ == "__main__":
    main()
