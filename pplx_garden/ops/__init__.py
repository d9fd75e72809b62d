"""Expert-side compute ops for the fused MoE layer (block-scaled fp8 grouped GEMM)."""

from pplx_garden.ops.grouped_gemm import (
    MODE_BF16 as MODE_BF16,
    MODE_BF16_SCATTER as MODE_BF16_SCATTER,
    MODE_SWIGLU_QUANT as MODE_SWIGLU_QUANT,
    SCALES_FP32 as SCALES_FP32,
    SCALES_POW2 as SCALES_POW2,
    dequantize_1x128 as dequantize_1x128,
    dequantize_128x128 as dequantize_128x128,
    grouped_fp8_gemm as grouped_fp8_gemm,
    quantize_1x128 as quantize_1x128,
    quantize_128x128 as quantize_128x128,
    round_scale_pow2 as round_scale_pow2,
)
from pplx_garden.ops.router import (
    topk_route as topk_route,
    topk_route_reference as topk_route_reference,
)
