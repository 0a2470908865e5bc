from .configuration_frac import FracConfig
from .modeling_frac import FracBlock, FracForCausalLM, FracMixer, FracModel

__all__ = ["FracConfig", "FracMixer", "FracBlock", "FracModel", "FracForCausalLM"]
