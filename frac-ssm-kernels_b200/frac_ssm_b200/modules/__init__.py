from .rmsnorm_gated import MambaRMSNormGated, rmsnorm_gated_fwd

__all__ = ["MambaRMSNormGated", "rmsnorm_gated_fwd"]
