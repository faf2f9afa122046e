"""Python face of the CPU oracle (oracle/quant_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU
baseline legs.  The product package (hidet_b200) never imports it.

All functions take and return numpy arrays.  See quant_oracle.c for what is restated from where and
for the parity status of each arithmetic.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import c_int, c_int64, c_void_p
from typing import Optional, Sequence, Tuple, Union

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
SOURCE = os.path.join(_DIR, 'quant_oracle.c')
LIBRARY = os.path.join(_DIR, 'libquant_oracle.so')
RCP_TABLE_FILE = os.path.join(_DIR, '..', 'tests', 'golden', 'rcp_approx_ftz_f32_of_f16.npy')

# Portable, strict IEEE build: the checker must give the same bits on every host.
STRICT_FLAGS = ['-O2', '-fPIC', '-shared', '-fopenmp', '-ffp-contract=off', '-fno-fast-math', '-fvisibility=hidden']
# The flags the reference's CPU backend compiles its generated code with
# (python/hidet/backend/build.py:326-338); used only for the timed CPU baseline.
REFERENCE_FLAGS = ['-O3', '-fPIC', '-shared', '-fopenmp', '-mavx2', '-m64', '-ffast-math', '-march=native', '-fvisibility=hidden']


def build(out: str = LIBRARY, flags: Sequence[str] = tuple(STRICT_FLAGS), force: bool = False) -> str:
    if force or not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(SOURCE):
        cmd = ['gcc', *flags, SOURCE, '-o', out, '-lm']
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if res.returncode != 0:
            raise RuntimeError('building the oracle failed:\n{}\n{}'.format(' '.join(cmd), res.stdout))
    return out


_libs = {}


def load(path: Optional[str] = None) -> ctypes.CDLL:
    if path is None:
        path = build()
    if path not in _libs:
        lib = ctypes.CDLL(path)
        lib.oracle_quantize_f16.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p]
        lib.oracle_dequantize_f16.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int]
        lib.oracle_qmatmul_f16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int64, c_int64]
        lib.oracle_qmatmul_f16_fused.argtypes = lib.oracle_qmatmul_f16.argtypes
        lib.oracle_quantize_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int]
        lib.oracle_dequantize_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int]
        lib.oracle_matmul_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]
        lib.oracle_qmatmul_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]
        lib.oracle_num_threads.restype = c_int
        lib.oracle_half_to_float.argtypes = [ctypes.c_uint16]
        lib.oracle_half_to_float.restype = ctypes.c_float
        lib.oracle_float_to_half.argtypes = [ctypes.c_float]
        lib.oracle_float_to_half.restype = ctypes.c_uint16
        lib.oracle_hdiv.argtypes = [ctypes.c_uint16, ctypes.c_uint16, c_void_p]
        lib.oracle_hdiv.restype = ctypes.c_uint16
        for name in ('oracle_quantize_f16', 'oracle_dequantize_f16', 'oracle_qmatmul_f16', 'oracle_qmatmul_f16_fused',
                     'oracle_quantize_f32', 'oracle_dequantize_f32', 'oracle_matmul_f32', 'oracle_qmatmul_f32'):
            getattr(lib, name).restype = None
        _libs[path] = lib
    return _libs[path]


_rcp_table: Optional[np.ndarray] = None
_rcp_table_loaded = False


def rcp_table() -> Optional[np.ndarray]:
    """uint32[65536]: bits of rcp.approx.ftz.f32(x) for every half bit pattern x, as measured on a
    B200 (tests/golden/make_rcp_table.py), or None if the measurement is not in the tree."""
    global _rcp_table, _rcp_table_loaded
    if not _rcp_table_loaded:
        _rcp_table_loaded = True
        if os.path.exists(RCP_TABLE_FILE):
            t = np.load(RCP_TABLE_FILE)
            assert t.dtype == np.uint32 and t.shape == (65536,)
            _rcp_table = np.ascontiguousarray(t)
    return _rcp_table


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(c_void_p)


def _q_bits(quant_type) -> int:
    name = np.dtype(quant_type).name if not isinstance(quant_type, str) else quant_type
    if name not in ('int8', 'int16'):
        raise ValueError('quant_type must be int8 or int16, got {!r}'.format(quant_type))
    return 8 if name == 'int8' else 16


def _as_2d(shape, dims) -> Tuple[int, int, int, list]:
    rank = len(shape)
    if isinstance(dims, int):
        dims = [dims]
    dims = sorted(d % rank for d in dims)
    keep = [i for i in range(rank) if i not in dims]
    scale_shape = [shape[i] for i in keep]
    n_red = int(np.prod([shape[i] for i in dims], dtype=np.int64))
    n_keep = int(np.prod(scale_shape, dtype=np.int64))
    if dims == list(range(rank - len(dims), rank)):
        return n_keep, n_red, 1, scale_shape
    if dims == list(range(len(dims))):
        return n_red, n_keep, 0, scale_shape
    raise NotImplementedError('oracle: dims must be leading or trailing')


def symmetric_quantize(w: np.ndarray, quant_type='int8', dims: Union[int, Sequence[int]] = -1, use_rcp_table: bool = True,
                       x86_fast_math: bool = False, lib: Optional[ctypes.CDLL] = None):
    """(wq, scale) as the reference computes them for a float16 (CUDA arithmetic) or float32 input.

    For float32, x86_fast_math=True gives the scale as the reference's -ffast-math x86 build evaluates it
    (absmax * (1/qmax)); False is the IEEE reading of the same expression (absmax / qmax)."""
    lib = lib or load()
    w = np.ascontiguousarray(w)
    rows, cols, reduce_dim, scale_shape = _as_2d(w.shape, dims)
    bits = _q_bits(quant_type)
    wq = np.empty(w.shape, dtype=np.int8 if bits == 8 else np.int16)
    scale = np.empty(scale_shape, dtype=w.dtype)
    if w.dtype == np.float16:
        table = rcp_table() if use_rcp_table else None
        lib.oracle_quantize_f16(_ptr(w), _ptr(wq), _ptr(scale), rows, cols, reduce_dim, bits, _ptr(table))
    elif w.dtype == np.float32:
        lib.oracle_quantize_f32(_ptr(w), _ptr(wq), _ptr(scale), rows, cols, reduce_dim, bits, 1 if x86_fast_math else 0)
    else:
        raise ValueError('oracle: unsupported dtype {}'.format(w.dtype))
    return wq, scale


def symmetric_dequantize(wq: np.ndarray, scale: np.ndarray, dims: Union[int, Sequence[int]] = -1,
                         lib: Optional[ctypes.CDLL] = None) -> np.ndarray:
    lib = lib or load()
    wq = np.ascontiguousarray(wq)
    scale = np.ascontiguousarray(scale)
    rows, cols, reduce_dim, scale_shape = _as_2d(wq.shape, dims)
    assert list(scale.shape) == scale_shape
    bits = _q_bits(wq.dtype)
    w = np.empty(wq.shape, dtype=scale.dtype)
    if scale.dtype == np.float16:
        lib.oracle_dequantize_f16(_ptr(wq), _ptr(scale), _ptr(w), rows, cols, reduce_dim, bits)
    elif scale.dtype == np.float32:
        lib.oracle_dequantize_f32(_ptr(wq), _ptr(scale), _ptr(w), rows, cols, reduce_dim, bits)
    else:
        raise ValueError('oracle: unsupported dtype {}'.format(scale.dtype))
    return w


def symmetric_quant_matmul(a: np.ndarray, wq: np.ndarray, scale: np.ndarray, layout: str = 'KN', k_begin: int = 0,
                           k_end: Optional[int] = None, fused: bool = False, lib: Optional[ctypes.CDLL] = None) -> np.ndarray:
    """float16 c = a @ dequant(wq, scale) summed over k in [k_begin, k_end).

    fused=False: the reference's dequantize-then-matmul value (weights rounded to half after scaling,
    exact sum); fused=True: exact integer sum scaled once in fp32, the value the new kernels aim at.
    float32 a / scale: the reference's x86 loop (KN layout, whole K)."""
    lib = lib or load()
    a = np.ascontiguousarray(a)
    wq = np.ascontiguousarray(wq)
    scale = np.ascontiguousarray(scale)
    k = a.shape[-1]
    m = int(np.prod(a.shape[:-1], dtype=np.int64))
    n = wq.shape[1] if layout == 'KN' else wq.shape[0]
    assert (wq.shape[0] if layout == 'KN' else wq.shape[1]) == k and scale.shape == (n,)
    if k_end is None:
        k_end = k
    c = np.empty(list(a.shape[:-1]) + [n], dtype=a.dtype)
    if a.dtype == np.float16:
        fn = lib.oracle_qmatmul_f16_fused if fused else lib.oracle_qmatmul_f16
        fn(_ptr(a), _ptr(wq), _ptr(scale), _ptr(c), m, n, k, 0 if layout == 'KN' else 1, k_begin, k_end)
    elif a.dtype == np.float32:
        assert layout == 'KN' and k_begin == 0 and k_end == k
        lib.oracle_qmatmul_f32(_ptr(a), _ptr(wq), _ptr(scale), _ptr(c), m, n, k)
    else:
        raise ValueError('oracle: unsupported dtype {}'.format(a.dtype))
    return c


def matmul_f32(a: np.ndarray, b: np.ndarray, lib: Optional[ctypes.CDLL] = None) -> np.ndarray:
    lib = lib or load()
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    c = np.empty((a.shape[0], b.shape[1]), dtype=np.float32)
    lib.oracle_matmul_f32(_ptr(a), _ptr(b), _ptr(c), a.shape[0], b.shape[1], a.shape[1])
    return c


def num_threads(lib: Optional[ctypes.CDLL] = None) -> int:
    return (lib or load()).oracle_num_threads()
