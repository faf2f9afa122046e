"""Calls the reference's own CUDA kernels, prebuilt under oracle/_ref/ by oracle/build_ref.py.

Test infrastructure only: the parity tests run these kernels on the GPU beside this repository's and
compare the results.  Each case library exports `hidet_launch(inputs..., outputs...)` taking raw device
pointers (python/hidet/drivers/build_task.py:68-106); the reference's runtime library supplies the stream
and scratch memory through callbacks that its Python side registers (python/hidet/ffi/callbacks.py) --
here they are served by torch allocations.
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import Dict, Optional, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, '_ref')

_ALLOC = ctypes.CFUNCTYPE(ctypes.c_uint64, ctypes.c_uint64)
_FREE = ctypes.CFUNCTYPE(None, ctypes.c_uint64)
_MEMSET = ctypes.CFUNCTYPE(None, ctypes.c_uint64, ctypes.c_int, ctypes.c_uint64)


def available() -> bool:
    return os.path.exists(os.path.join(REF_DIR, 'manifest.json'))


class ReferenceKernels:
    def __init__(self):
        import torch

        self.torch = torch
        self.manifest = json.load(open(os.path.join(REF_DIR, 'manifest.json')))
        self.cases = {c['name']: c for c in self.manifest['cases']}
        self.runtime = ctypes.CDLL(os.path.join(REF_DIR, self.manifest['runtime']), mode=ctypes.RTLD_GLOBAL)
        self.runtime.hidet_get_last_error.restype = ctypes.c_char_p
        self.runtime.register_callback.argtypes = [ctypes.c_char_p, ctypes.c_void_p]
        self.runtime.set_cuda_stream.argtypes = [ctypes.c_void_p]
        self.runtime.use_torch_cuda_stream.argtypes = [ctypes.c_bool]
        self._storage: Dict[int, 'torch.Tensor'] = {}
        self._libs: Dict[str, ctypes.CDLL] = {}

        def allocate(nbytes):
            t = torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device='cuda')
            self._storage[t.data_ptr()] = t
            return t.data_ptr()

        def free(ptr):
            self._storage.pop(int(ptr), None)

        def memset(ptr, value, nbytes):
            self._storage[int(ptr)][:int(nbytes)].fill_(int(value) & 0xff)

        self._callbacks = (_ALLOC(allocate), _FREE(free), _MEMSET(memset))   # kept alive with the object
        for name, cb in zip((b'allocate_cuda_storage', b'free_cuda_storage', b'cuda_memset'), self._callbacks):
            self.runtime.register_callback(name, ctypes.cast(cb, ctypes.c_void_p))
        self.runtime.use_torch_cuda_stream(False)

    _DEFAULTS = {'wtype': 'float16', 'qtype': 'int8'}

    def find(self, kind: str, **params) -> Optional[str]:
        for c in self.manifest['cases']:
            if c['kind'] == kind and all(c.get(k, self._DEFAULTS.get(k)) == v for k, v in params.items()):
                return c['name']
        return None

    def launch(self, name: str, *tensors) -> None:
        """hidet_launch of one case on torch's current stream; raises with the reference's own message."""
        for t in tensors:
            assert t.is_cuda and t.is_contiguous()
        self.launch_pointers(name, *[t.data_ptr() for t in tensors])

    def launch_pointers(self, name: str, *pointers) -> None:
        """The same with raw device addresses (0 for a null pointer)."""
        torch = self.torch
        lib = self._libs.get(name)
        if lib is None:
            lib = self._libs[name] = ctypes.CDLL(os.path.join(REF_DIR, self.cases[name]['file']))
            lib.hidet_launch.restype = None
        self.runtime.set_cuda_stream(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        lib.hidet_launch(*[ctypes.c_void_p(p) for p in pointers])
        err = self.runtime.hidet_get_last_error()
        if err:
            raise RuntimeError('reference kernel {}: {}'.format(name, err.decode()))
        torch.cuda.current_stream().synchronize()

    # ---- the operators of the path, by the reference's names ----
    def symmetric_quantize(self, w, dims: int, quant_type: str = 'int8') -> Tuple['torch.Tensor', 'torch.Tensor']:
        torch = self.torch
        rows, cols = w.shape
        wtype = {torch.float16: 'float16', torch.bfloat16: 'bfloat16'}[w.dtype]
        name = self.find('quantize', rows=rows, cols=cols, dims=dims, wtype=wtype, qtype=quant_type)
        if name is None:
            raise KeyError('no reference kernel was built for quantize {} -> {} {}x{} dims={}'.format(wtype, quant_type, rows, cols, dims))
        wq = torch.empty(rows, cols, dtype=getattr(torch, quant_type), device='cuda')
        scale = torch.empty(cols if dims == 0 else rows, dtype=w.dtype, device='cuda')
        self.launch(name, w, wq, scale)
        return wq, scale

    def symmetric_dequantize(self, wq, scale, dims: int):
        torch = self.torch
        rows, cols = wq.shape
        wtype = {torch.float16: 'float16', torch.bfloat16: 'bfloat16'}[scale.dtype]
        qtype = {torch.int8: 'int8', torch.int16: 'int16'}[wq.dtype]
        name = self.find('dequantize', rows=rows, cols=cols, dims=dims, wtype=wtype, qtype=qtype)
        if name is None:
            raise KeyError('no reference kernel was built for dequantize {} {} {}x{} dims={}'.format(wtype, qtype, rows, cols, dims))
        w = torch.empty(rows, cols, dtype=scale.dtype, device='cuda')
        self.launch(name, wq, scale, w)
        return w

    def quant_matmul(self, a, wq, scale, kind: str = 'matmul_f16_i8'):
        """kind='matmul_f16_i8': the tensor-core kernel (one split-K part); 'matmul_generic': the auto-scheduled one."""
        torch = self.torch
        m, k = a.shape
        n = wq.shape[1]
        name = self.find(kind, m=m, k=k, n=n)
        if name is None:
            raise KeyError('no reference kernel was built for {} {}x{}x{}'.format(kind, m, k, n))
        c = torch.empty(m, n, dtype=torch.float16, device='cuda')
        self.launch(name, a, wq, scale, c)
        return c
