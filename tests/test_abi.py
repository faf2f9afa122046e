"""The C ABI and the host layer, without a GPU: the library loads, exports what the header declares,
reports errors the documented way, and the host layer validates like the reference."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT

import hidet_b200
from hidet_b200 import ffi


def _declared_symbols():
    text = open(os.path.join(ROOT, 'include', 'hidet_b200q.h')).read()
    return sorted(set(re.findall(r'B200Q_API\s+[\w\s\*]+?\b(b200q_\w+)\s*\(', text)))


def test_header_symbols_are_exported_and_bound():
    declared = _declared_symbols()
    assert len(declared) >= 8
    lib = ctypes.CDLL(ffi.library_path())
    for name in declared:
        assert hasattr(lib, name), '{} is declared but not exported'.format(name)
        assert name in ffi.SIGNATURES, '{} has no ctypes signature in hidet_b200.ffi'.format(name)
    assert sorted(ffi.SIGNATURES) == declared


def test_version_and_error_state():
    assert ffi.version() == 100
    assert ffi.get_last_error() is None
    # argument validation happens before any CUDA call, so it can be exercised on a CPU-only host
    with pytest.raises(ffi.BackendException) as e:
        ffi.func('b200q_symmetric_quantize')(None, None, None, 4, 4, 99, 0, 0, None)
    assert 'unknown float type 99' in str(e.value) and e.value.status == ffi.INVALID_ARGUMENT
    assert ffi.get_last_error() is None  # read-and-clear
    with pytest.raises(ffi.BackendException) as e:
        ffi.func('b200q_qlinear_f16_i8')(None, None, None, None, 4, -1, 4, 0, None, 0, None)
    assert 'negative size' in str(e.value)
    with pytest.raises(ffi.BackendException) as e:
        ffi.func('b200q_qlinear_f16_i8_parts')(1, 1, 1, 1, 4, 4, 4, 0, None)
    assert 'k_parts' in str(e.value)


def test_workspace_query_is_pure():
    ws = ffi.func('b200q_qlinear_workspace_bytes')
    assert ws(0, 4096, 4096, 0) == 0
    # a square projection is split inside clusters and needs no scratch; a narrow, deep one is split
    # over several clusters that meet in the workspace
    assert ws(16, 4096, 4096, 0) == 0
    small = ws(1, 1024, 28672, 0)
    big = ws(16, 1024, 28672, 0)
    assert 0 < small <= big < 64 * 1024 * 1024


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(ffi, '_lib', None)
    monkeypatch.setattr(ffi, '_funcs', {})
    monkeypatch.setattr(ffi, 'library_search_paths', lambda: [str(tmp_path / 'nope.so')])
    with pytest.raises(ffi.BackendException) as e:
        ffi.func('b200q_version')
    assert 'no other implementation' in str(e.value)


def test_cpu_tensors_are_rejected_not_computed():
    w = torch.zeros(8, 8, dtype=torch.float16)
    with pytest.raises(ffi.BackendException):
        hidet_b200.symmetric_quantize(w, 'int8', dims=0)
    with pytest.raises(ffi.BackendException):
        hidet_b200.symmetric_quant_matmul(w, w.to(torch.int8), w[0])


def test_dims_normalisation():
    from hidet_b200.quant.symmetric import _as_2d, _normalize_dims

    assert _normalize_dims(-1, 2) == [1] and _normalize_dims([0], 2) == [0]
    assert _as_2d([64, 48], [0]) == (64, 48, 0, [48])
    assert _as_2d([64, 48], [1]) == (64, 48, 1, [64])
    assert _as_2d([2, 3, 8], [2]) == (6, 8, 1, [2, 3])
    assert _as_2d([2, 3, 8], [0]) == (2, 24, 0, [3, 8])
    assert _as_2d([5], [0]) == (1, 5, 1, [])
    with pytest.raises(NotImplementedError):
        _as_2d([2, 3, 8], [1])
    with pytest.raises(ValueError):
        _normalize_dims(2, 2)
