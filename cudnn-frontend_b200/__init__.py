"""B200-native MoE grouped-GEMM hot path behind cudnn-frontend's Python signatures.

Public names mirror what the reference exports from its package root through lazy attributes
(python/cudnn/__init__.py:241-281):

    GroupedGemmSwigluSm100, grouped_gemm_swiglu_wrapper_sm100
    GroupedGemmQuantSm100, grouped_gemm_quant_wrapper_sm100
    DiscreteGroupedGemmSwigluSm100, discrete_grouped_gemm_swiglu_wrapper_sm100
    GroupedGemmGluSm100, grouped_gemm_glu_wrapper_sm100      (unified FC1: swiglu / geglu, bias)
    GroupedGemmDswigluSm100, grouped_gemm_dswiglu_wrapper_sm100  (backward of FC1's activation)
    DiscreteGroupedGemmDswigluSm100, discrete_grouped_gemm_dswiglu_wrapper_sm100
    GroupedGemmWgradSm100, grouped_gemm_wgrad_wrapper_sm100      (weight gradient: the experts split K)

plus what the reference does not have: ``quantize_mxfp8`` (activation quantiser), the routing
helpers of ``moe`` and the expert-parallel layer ``ExpertParallelMoE``.
"""

__version__ = "0.1.0"

_LAZY = {
    "GroupedGemmSwigluSm100": "grouped_gemm_swiglu",
    "grouped_gemm_swiglu_wrapper_sm100": "grouped_gemm_swiglu",
    "GroupedGemmQuantSm100": "grouped_gemm_quant",
    "grouped_gemm_quant_wrapper_sm100": "grouped_gemm_quant",
    "DiscreteGroupedGemmSwigluSm100": "discrete_grouped_gemm_swiglu",
    "discrete_grouped_gemm_swiglu_wrapper_sm100": "discrete_grouped_gemm_swiglu",
    "GroupedGemmGluSm100": "grouped_gemm_glu",
    "grouped_gemm_glu_wrapper_sm100": "grouped_gemm_glu",
    "GroupedGemmDswigluSm100": "grouped_gemm_dswiglu",
    "grouped_gemm_dswiglu_wrapper_sm100": "grouped_gemm_dswiglu",
    "DiscreteGroupedGemmDswigluSm100": "grouped_gemm_dswiglu",
    "discrete_grouped_gemm_dswiglu_wrapper_sm100": "grouped_gemm_dswiglu",
    "GroupedGemmWgradSm100": "grouped_gemm_wgrad",
    "grouped_gemm_wgrad_wrapper_sm100": "grouped_gemm_wgrad",
    "TupleDict": "api_base",
    "quantize_mxfp8": "ops",
    "quantize_mxfp8_out": "ops",
    "empty_sf": "ops",
    "route": "moe",
    "scatter_rows": "moe",
    "combine_rows": "moe",
    "interleave_gate_up": "moe",
    "ExpertParallelMoE": "ep_layer",
}


def __getattr__(name):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    import importlib

    return getattr(importlib.import_module(f"{__name__}.{mod}"), name)


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
