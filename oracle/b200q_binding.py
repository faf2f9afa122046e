"""The reference-side binding of libhidet_b200q.so: a task of the reference (hidet-org/hidet) whose CUDA
implementation calls this repository's library.

This is the module a maintainer of the reference would add next to python/hidet/graph/ops/quant/matmul.py.  Here it
is test infrastructure: oracle/build_ref.py imports the reference, lets it generate and compile this task exactly
as it builds its own (same code generator, same nvcc flags), and tests/test_reference_binding_gpu.py calls the
resulting `hidet_launch` on the GPU.  (No `from __future__ import annotations` in this file: the reference's
script front end reads the annotations of `launch` as objects.)
"""
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INCLUDE_DIR = os.path.join(ROOT, 'include')
LIBRARY_DIR = os.path.join(ROOT, 'hidet_b200', 'lib')


def b200q_task(hidet, a, b, scale):
    """SymmetricQuantizedMatmulTask (python/hidet/graph/ops/quant/matmul.py:24-74: same inputs, output and compute
    definition, so shape inference and graph passes see the operator they know) whose CUDA implementation is not
    scheduled by the reference but handed to libhidet_b200q.so: `launch` asks the reference's runtime for the stream
    and the workspace and calls b200q_qlinear_f16_i8, registered as a primitive function the way the cuBLAS
    wrappers are (python/hidet/graph/ops/matmul/matmul_cublas.py:49-90, python/hidet/ir/library/cuda/cublas/regs.py);
    a failure is forwarded to hidet_set_last_error, where the reference's Python side looks after every call
    (python/hidet/runtime/compiled_module.py:79-102)."""
    from hidet.graph.ops.quant.matmul import SymmetricQuantizedMatmulTask
    from hidet.ir.dtypes import boolean, float16, int8, int32, int64
    from hidet.ir.primitives.func import call_primitive_func, is_primitive_function, register_primitive_function
    from hidet.ir.primitives.runtime import get_cuda_stream, request_cuda_workspace
    from hidet.ir.stmt import BlackBoxStmt
    from hidet.ir.type import FuncType, void_p
    from hidet.lang import attrs

    if not is_primitive_function('b200q.qlinear_f16_i8'):
        register_primitive_function('b200q.qlinear_workspace_bytes', FuncType([int64, int64, int64, int32], int64),
                                    codegen_name='b200q_qlinear_workspace_bytes')
        register_primitive_function('b200q.qlinear_f16_i8',
                                    FuncType([void_p, void_p, void_p, void_p, int64, int64, int64, int32, void_p, int64, void_p], int32),
                                    codegen_name='b200q_qlinear_f16_i8')

    class B200QuantizedMatmulTask(SymmetricQuantizedMatmulTask):
        def __init__(self, a, b, scale):
            super().__init__(a, b, scale)
            self.name = 'b200q_symmetric_quantized_matmul'   # caches key on the task name

        def implement_cuda(self, working_dir):
            m, k = [int(v) for v in self.inputs[0].type.shape]
            n = int(self.inputs[1].type.shape[1])

            with hidet.script_module() as script_module:

                @hidet.script
                def launch(a: float16[m, k], b: int8[k, n], scale: float16[n], c: float16[m, n]):
                    attrs.func_kind = 'public'

                    ws_bytes = call_primitive_func('b200q.qlinear_workspace_bytes', [int64(m), int64(n), int64(k), int32(0)])
                    ws = request_cuda_workspace(ws_bytes, boolean(True))
                    status = call_primitive_func('b200q.qlinear_f16_i8', [a, b, scale, c, int64(m), int64(n), int64(k), int32(0), ws, ws_bytes,
                                                                          get_cuda_stream()])
                    BlackBoxStmt('if ({} != 0) hidet_set_last_error(b200q_get_last_error());', status)

            ir_module = script_module.ir_module()
            ir_module.include_headers.append('hidet_b200q.h')
            ir_module.include_dirs.append(INCLUDE_DIR)
            ir_module.linking_dirs.append(LIBRARY_DIR)
            ir_module.linking_libs.append(':libhidet_b200q.so')
            return ir_module

    return B200QuantizedMatmulTask(a, b, scale)


