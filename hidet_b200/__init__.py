"""hidet_b200: Hidet's weight-only int8 quantized linear path on B200 (sm_100a).

The public names follow the reference (hidet.ops.symmetric_quantize, hidet.ops.symmetric_dequantize,
hidet.ops.quant.*); tensors are CUDA torch tensors and every computation runs in the hand-written
kernels of libhidet_b200q.so, reached through ctypes.  Importing the package touches neither CUDA
nor the library.
"""
from . import ffi
from . import quant
from . import graph
from .cuda_graph import CudaGraph
from .quant import (
    symmetric_quantize,
    symmetric_dequantize,
    symmetric_dequantize_take,
    symmetric_quant_matmul,
    symmetric_quant_matmul_f16_i8,
    symmetric_quant_matmul_atomic_f16_i8,
)

__version__ = '0.1.0'
