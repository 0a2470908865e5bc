"""Model configuration with the reference's field names and defaults
(`frac_ssm/models/configuration_frac.py:8-97`), as a plain object: the B200 model classes do not
depend on the `transformers` package."""

from __future__ import annotations


class FracConfig:
    model_type = "frac"

    def __init__(self, vocab_size=32000, hidden_size=768, intermediate_size=None, num_hidden_layers=24,
                 num_attention_heads=12, hidden_act="silu", max_position_embeddings=32768,
                 initializer_range=0.02, rms_norm_eps=1e-6, use_cache=True, pad_token_id=0, bos_token_id=1,
                 eos_token_id=2, tie_word_embeddings=True, frac_expand=2.0, frac_num_modes=8,
                 frac_conv_kernel=4, frac_dt_min=1e-4, frac_dt_max=1.0, frac_alpha_min=0.20,
                 frac_alpha_max=0.95, frac_tau_min=1.0, frac_tau_max=65536.0, frac_chunk_size=32,
                 frac_lambda_min=0.25, frac_lambda_max=4.0, frac_residual_read_init=-2.0,
                 frac_write_scale_init=0.25, frac_gate_bias_init=0.0, frac_conv_bias=True,
                 frac_head_dim=None, **unused):
        if hidden_act not in ("silu", "swish"):
            raise ValueError("only the silu/swish activation is supported")
        if frac_chunk_size < 16 or frac_chunk_size & (frac_chunk_size - 1):
            raise ValueError(f"frac_chunk_size must be a power of two greater than or equal to 16, got {frac_chunk_size}.")
        inner = int(hidden_size * frac_expand) if intermediate_size is None else intermediate_size
        if frac_head_dim is None:
            if inner % num_attention_heads:
                raise ValueError(f"intermediate_size={inner} must be divisible by num_attention_heads={num_attention_heads}.")
            frac_head_dim = inner // num_attention_heads
        elif frac_head_dim * num_attention_heads != inner:
            raise ValueError("frac_head_dim * num_attention_heads must equal intermediate_size. "
                             f"Got {frac_head_dim} * {num_attention_heads} != {inner}.")
        self.vocab_size, self.hidden_size, self.intermediate_size = vocab_size, hidden_size, inner
        self.num_hidden_layers, self.num_attention_heads = num_hidden_layers, num_attention_heads
        self.hidden_act, self.max_position_embeddings = hidden_act, max_position_embeddings
        self.initializer_range, self.rms_norm_eps, self.use_cache = initializer_range, rms_norm_eps, use_cache
        self.pad_token_id, self.bos_token_id, self.eos_token_id = pad_token_id, bos_token_id, eos_token_id
        self.tie_word_embeddings = tie_word_embeddings
        self.frac_expand, self.frac_num_modes, self.frac_conv_kernel = frac_expand, frac_num_modes, frac_conv_kernel
        self.frac_dt_min, self.frac_dt_max = frac_dt_min, frac_dt_max
        self.frac_alpha_min, self.frac_alpha_max = frac_alpha_min, frac_alpha_max
        self.frac_tau_min, self.frac_tau_max = frac_tau_min, frac_tau_max
        self.frac_chunk_size = frac_chunk_size
        self.frac_lambda_min, self.frac_lambda_max = frac_lambda_min, frac_lambda_max
        self.frac_residual_read_init, self.frac_write_scale_init = frac_residual_read_init, frac_write_scale_init
        self.frac_gate_bias_init, self.frac_conv_bias, self.frac_head_dim = frac_gate_bias_init, frac_conv_bias, frac_head_dim

    def to_dict(self):
        return dict(self.__dict__)
