"""Mirror of hidet.graph.ops.quant (python/hidet/graph/ops/quant/__init__.py:12-15)."""
from .symmetric import symmetric_quantize, symmetric_dequantize, symmetric_dequantize_take
from .matmul import interleave_gate_up, symmetric_quant_matmul, symmetric_quant_matmul_f16_i8, symmetric_quant_matmul_atomic_f16_i8
from .subbyte import cast_f16_to_u4, cast_u4_to_f16, preprocess_weight, w4a16_linear, FpAIntBGemm
