"""Graph-level half of the path: operator objects, resolve rules, the quantization pass over
torch.fx graphs and the torch.compile backend (see the module docstrings for the reference files each
part mirrors)."""
from .operators import (
    Operator,
    SymmetricQuantizationOp,
    SymmetricDeQuantizationOp,
    SymmetricQuantizedMatmulOp,
    SymmetricQuantizedMatmulF16I8Op,
)
from .transforms import PassContext, ResolveRule, register_resolve_rule, SubgraphRewriteRule, optimize, resolve_operator
from .patterns import (
    default_patterns,
    symmetric_linear_patterns,
    symmetric_embedding_quantize_patterns,
    SymmetricLinearQuantizePattern,
    SymmetricLinearQuantizePatternR,
    SymmetricLinearQuantizePatternL,
    SymmetricQuantizeMatmulFused,
    SymmetricEmbeddingQuantizePattern,
    QuantizedLinearEpilogueFusion,
    QuantizedLinearConcat,
    quantized_matmul,
    quantized_linear_nk,
    quantized_embedding,
    dequantized_weight,
)
from .dynamo_backend import hidet_b200_backend, register
