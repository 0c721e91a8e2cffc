"""es_b200: B200-native (sm_100a) MoE grouped-GEMM operators behind the op surface of `expert_specialization`.

    from expert_specialization_moe_b200 import (
        es_fp8_blockwise_scaled_grouped_mm,
        es_sm100_mxfp8_blockscaled_grouped_mm,
        es_sm100_mxfp8_blockscaled_grouped_quant,
    )

mirrors `from expert_specialization import ...` (reference: expert_specialization/__init__.py:1-3).
"""
from .ops import (  # noqa: F401
    es_fp8_blockwise_scaled_grouped_mm,
    es_sm100_mxfp8_blockscaled_grouped_mm,
    es_sm100_mxfp8_blockscaled_grouped_quant,
    es_sm100_mxfp8_silu_mul_grouped_quant,
)
