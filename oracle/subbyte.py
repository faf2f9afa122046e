"""CPU restatement of the reference's 4-bit weight path (numpy).

TEST INFRASTRUCTURE ONLY: imported by tests/; the product package (hidet_b200) never imports it.

What is restated from where:
* storage of a sub-byte type: element i of a row lives in bits nbits * (i % per) .. of storage unit i / per, low bits
  first (python/hidet/transforms/lower_integer_subbyte.py:103-113, `(base[idx] >> (offset * nbits)) & mask`);
* cast f16 -> u4: C conversion to int, low four bits (tests/cute_kernel/quantized_linear.py:226-267, `cast(tr_wi, u4)`);
* the linear: c = a @ (scale * (b - zeros)) per group of `group_size` k rows, or a @ (scale * b) without zero
  points (tests/cute_kernel/test_quant_linear.py:68-85, the check the reference's own test makes; its kernel forms
  `scale * (f16(b) - zeros)` in f16 and accumulates the products, tests/cute_kernel/quantized_linear.py:1044-1047).

Parity: the reference's kernel is written in its CuTe dialect and is compiled by its Python compiler at run time; it
cannot be built from source files alone, and its test holds no stored vectors (it compares with `a @ b` computed by
torch on small-integer data, where every product and sum is exact).  The oracle is pinned by that property:
tests/test_subbyte_cpu.py checks that on the reference's own data distribution the restatement equals the exact
integer result, and the nibble order against hand-written bytes.
"""
from __future__ import annotations

from typing import Optional

import numpy as np


def pack_u4(values: np.ndarray) -> np.ndarray:
    """[rows, cols] numbers -> uint8 [rows, cols / 2]: C conversion to int, low four bits, low nibble first."""
    v = np.asarray(values)
    if v.ndim != 2 or v.shape[1] % 2 != 0:
        raise ValueError('expect a matrix with an even number of columns')
    codes = (np.trunc(v.astype(np.float64)).astype(np.int64) & 15).astype(np.uint8)
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)


def unpack_u4(packed: np.ndarray) -> np.ndarray:
    """uint8 [rows, cols / 2] -> uint8 codes [rows, cols]."""
    p = np.asarray(packed).view(np.uint8) if np.asarray(packed).dtype != np.uint8 else np.asarray(packed)
    out = np.empty((p.shape[0], p.shape[1] * 2), dtype=np.uint8)
    out[:, 0::2] = p & 15
    out[:, 1::2] = p >> 4
    return out


def dequantize(codes: np.ndarray, scale: np.ndarray, zeros: Optional[np.ndarray], group_size: int, f16_steps: bool = False) -> np.ndarray:
    """w[k, n] = scale[k / G, n] * (q[k, n] - zeros[k / G, n]); float64, or rounded to f16 after the subtraction and
    after the product as the reference's kernel does (f16_steps)."""
    k, n = codes.shape
    s = np.repeat(np.asarray(scale, dtype=np.float16), group_size, axis=0)[:k]
    q = codes.astype(np.float16)
    if f16_steps:
        d = q if zeros is None else (q - np.repeat(np.asarray(zeros, dtype=np.float16), group_size, axis=0)[:k]).astype(np.float16)
        return (s * d).astype(np.float16).astype(np.float64)
    d = q.astype(np.float64)
    if zeros is not None:
        d = d - np.repeat(np.asarray(zeros, dtype=np.float16), group_size, axis=0)[:k].astype(np.float64)
    return s.astype(np.float64) * d


def w4a16_linear(a: np.ndarray, packed: np.ndarray, scale: np.ndarray, zeros: Optional[np.ndarray], group_size: int,
                 f16_steps: bool = False) -> np.ndarray:
    """c[M, N] in float64 (the caller rounds)."""
    w = dequantize(unpack_u4(packed), scale, zeros, group_size, f16_steps)
    return np.asarray(a, dtype=np.float16).astype(np.float64) @ w
