from .compute_params import compute_params_from_projections, frac_compute_scan_params
from .output_mix import (frac_skip_mix, scan_epilogue, scan_epilogue_apply, scan_epilogue_sumsq,
                         scan_layer, scan_layer_gated, scan_layer_norm, scan_layer_sumsq,
                         scan_layer_supported, skip_mix)

__all__ = ["frac_compute_scan_params", "frac_skip_mix", "compute_params_from_projections",
           "skip_mix", "scan_epilogue", "scan_epilogue_sumsq", "scan_epilogue_apply", "scan_layer",
           "scan_layer_gated", "scan_layer_norm", "scan_layer_sumsq", "scan_layer_supported"]
