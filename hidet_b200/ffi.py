"""ctypes binding of ``libhidet_b200q.so``.

Mirrors how the reference reaches its own native code: the library is loaded once
(python/hidet/ffi/ffi.py:32-69), functions are looked up with explicit argument types through
``get_func`` and every call is followed by a check of the library's thread-local error message, which
is raised as ``BackendException`` (python/hidet/ffi/ffi.py:71-99).

There is no fallback: if the library is absent, or lacks a symbol, the first use raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p
from typing import Callable, Dict, List, Optional

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIBRARY_NAME = 'libhidet_b200q.so'


class BackendException(Exception):
    """A call into libhidet_b200q.so failed.  Same name and role as hidet.ffi.ffi.BackendException."""

    def __init__(self, message: str, status: int = -1):
        super().__init__(message)
        self.status = status


# status codes of include/hidet_b200q.h
OK = 0
INVALID_ARGUMENT = 1
UNSUPPORTED = 2
WORKSPACE_TOO_SMALL = 3
CUDA_ERROR = 4
KERNEL_TIMEOUT = 5

# enums of include/hidet_b200q.h
F16, BF16, F32 = 0, 1, 2
I8, I16 = 0, 1
LAYOUT_KN, LAYOUT_NK = 0, 1
ACT_NONE, ACT_SILU_MUL = 0, 1


class Epilogue(ctypes.Structure):
    """b200q_epilogue of include/hidet_b200q.h."""

    _fields_ = [('bias', c_void_p), ('residual', c_void_p), ('ldr', c_int64), ('activation', c_int)]

_lib: Optional[ctypes.CDLL] = None
_funcs: Dict[str, Callable] = {}


def library_search_paths() -> List[str]:
    paths = []
    env = os.environ.get('HIDET_B200Q_LIBRARY')
    if env:
        paths.append(env)
    paths.append(os.path.join(_PKG_DIR, 'lib', LIBRARY_NAME))
    return paths


def library_path() -> str:
    for p in library_search_paths():
        if os.path.exists(p):
            return p
    raise BackendException(
        '{} not found (looked in: {}). Build it with `python -m hidet_b200.build`; '
        'there is no other implementation to fall back to.'.format(LIBRARY_NAME, ', '.join(library_search_paths()))
    )


def load_library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = library_path()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise BackendException('failed to load {}: {}'.format(path, e)) from e
        _lib.b200q_get_last_error.restype = c_char_p
        _lib.b200q_get_last_error.argtypes = []
    return _lib


def get_last_error() -> Optional[str]:
    """Read and clear the calling thread's error message (None if there is none)."""
    msg = load_library().b200q_get_last_error()
    text = msg.decode('utf-8') if msg else ''
    return text if text else None


def get_func(func_name: str, arg_types: List, restype=c_int, status_checked: bool = True) -> Callable:
    """Look up an entry point and wrap it so that a failed call raises BackendException."""
    key = func_name
    if key in _funcs:
        return _funcs[key]
    lib = load_library()
    try:
        func = getattr(lib, func_name)
    except AttributeError as e:
        raise BackendException('{} does not export {}'.format(library_path(), func_name)) from e
    func.argtypes = arg_types
    func.restype = restype

    if status_checked:

        def func_with_check(*args):
            status = func(*args)
            if status != OK:
                msg = get_last_error() or 'status {}'.format(status)
                raise BackendException('Calling {} failed with error:\n{}'.format(func_name, msg), status)
            return status

        wrapped = func_with_check
    else:
        wrapped = func
    _funcs[key] = wrapped
    return wrapped


# Every symbol include/hidet_b200q.h declares, with its ctypes signature.
SIGNATURES = {
    'b200q_version': ([], c_int, False),
    'b200q_get_last_error': ([], c_char_p, False),
    'b200q_check_status': ([], c_int, True),
    'b200q_symmetric_quantize': ([c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_void_p], c_int, True),
    'b200q_symmetric_dequantize': ([c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_void_p], c_int, True),
    'b200q_embedding_dequantize': (
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_void_p],
        c_int,
        True,
    ),
    'b200q_qlinear_f16_u4_workspace_bytes': ([c_int64, c_int64, c_int64, c_int64], c_size_t, False),
    'b200q_qlinear_f16_u4': (
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p],
        c_int,
        True,
    ),
    'b200q_u4_pack': ([c_void_p, c_void_p, c_int64, c_int64, c_void_p], c_int, True),
    'b200q_u4_unpack': ([c_void_p, c_void_p, c_int64, c_int64, c_void_p], c_int, True),
    'b200q_qlinear_workspace_bytes': ([c_int64, c_int64, c_int64, c_int], c_size_t, False),
    'b200q_qlinear_f16_i8': (
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_size_t, c_void_p],
        c_int,
        True,
    ),
    'b200q_qlinear_f16_i8_fused': (
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_size_t, c_void_p],
        c_int,
        True,
    ),
    'b200q_qlinear_f16_i8_to_peers': (
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p],
        c_int,
        True,
    ),
    'b200q_qlinear_f16_i8_to_multicast': (
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p],
        c_int,
        True,
    ),
    'b200q_push_columns': ([c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_void_p], c_int, True),
    'b200q_qlinear_static_scratch_bytes': ([], c_size_t, False),
    'b200q_qlinear_f16_i8_static': ([c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p], c_int, True),
    'b200q_qlinear_f16_i8_parts': ([c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p], c_int, True),
}


def func(name: str) -> Callable:
    arg_types, restype, checked = SIGNATURES[name]
    return get_func(name, arg_types, restype, checked)


def version() -> int:
    return func('b200q_version')()
