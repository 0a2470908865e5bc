"""The B200 model classes mirror the reference's module tree: a reference state_dict loads strictly."""

import os

import pytest
import torch


@pytest.mark.parametrize("name", ["model_tiny", "model_wide"])
def test_reference_state_dict_loads_strictly(golden_dir, name):
    from frac_ssm_b200.models import FracConfig, FracForCausalLM
    g = torch.load(os.path.join(golden_dir, name + ".pt"), weights_only=False)
    model = FracForCausalLM(FracConfig(**g["config"]))
    missing, unexpected = model.load_state_dict(g["state_dict"], strict=True)
    assert not missing and not unexpected
    assert model.lm_head.weight is model.model.embed_tokens.weight      # tied, as in the reference


def test_config_validation_matches_reference_messages():
    from frac_ssm_b200.models import FracConfig
    with pytest.raises(ValueError, match="power of two greater than or equal to 16"):
        FracConfig(frac_chunk_size=24)
    with pytest.raises(ValueError, match="must be divisible by"):
        FracConfig(hidden_size=100, num_attention_heads=7)
    with pytest.raises(ValueError, match="must equal intermediate_size"):
        FracConfig(hidden_size=64, num_attention_heads=2, frac_head_dim=48)
    cfg = FracConfig(hidden_size=768, num_attention_heads=24, frac_num_modes=128, frac_chunk_size=256)
    assert cfg.intermediate_size == 1536 and cfg.frac_head_dim == 64
