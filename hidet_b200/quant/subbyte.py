"""4-bit weights with group scales and zero points (w4a16): the operations of the reference's CuTe test programs
(tests/cute_kernel/quantized_linear.py, tests/cute_kernel/test_quant_linear.py) under the same names.

    bq = cast_f16_to_u4(b)                       # [K, N] f16 of integers 0..15 -> packed codes, [K, N / 8] int32
    linear = w4a16_linear('name', k, n, group_size, with_zp=True)
    c = linear(a, bq, scale, zeros)              # a [M, K] f16; scale, zeros [K / group_size, N] f16

The reference's `preprocess_weight` permutes the packed weight into a layout private to its kernel; the kernel
here reads the plain packed matrix, so `preprocess_weight` is the identity.
"""
from __future__ import annotations

import torch

from .. import ffi
from ..runtime import current_stream_ptr, require_cuda, workspaces


def cast_f16_to_u4(t: torch.Tensor) -> torch.Tensor:
    """f16 [rows, cols] -> u4 codes, eight per int32 (tests/cute_kernel/quantized_linear.py:226-267): C conversion to
    int, low four bits, element i of a row in bits 4 (i % 8) .. + 3 of word i / 8."""
    require_cuda(t, 't')
    if t.dtype != torch.float16 or t.dim() != 2 or t.shape[1] % 8 != 0:
        raise ValueError('expect a float16 matrix whose row length is a multiple of 8, got {} {}'.format(t.dtype, list(t.shape)))
    t = t.contiguous()
    rows, cols = t.shape
    out = torch.empty((rows, cols // 8), dtype=torch.int32, device=t.device)
    with torch.cuda.device(t.device):
        ffi.func('b200q_u4_pack')(t.data_ptr(), out.data_ptr(), rows, cols, current_stream_ptr(t.device))
    return out


def cast_u4_to_f16(t: torch.Tensor) -> torch.Tensor:
    """Packed u4 codes [rows, cols / 8] int32 -> f16 [rows, cols] (tests/cute_kernel/quantized_linear.py:181-223)."""
    require_cuda(t, 't')
    if t.dim() != 2:
        raise ValueError('expect a matrix of packed codes')
    t = t.contiguous()
    rows = t.shape[0]
    cols = t.shape[1] * t.element_size() * 2
    out = torch.empty((rows, cols), dtype=torch.float16, device=t.device)
    with torch.cuda.device(t.device):
        ffi.func('b200q_u4_unpack')(t.data_ptr(), out.data_ptr(), rows, cols, current_stream_ptr(t.device))
    return out


def preprocess_weight(weight: torch.Tensor) -> torch.Tensor:
    """The kernel reads the plain packed matrix: nothing to do (the reference permutes for its own kernel,
    tests/cute_kernel/quantized_linear.py:269-343)."""
    return weight


class FpAIntBGemm:
    """c = a @ (scale * (b - zeros)) per group of `group_size` k rows, b in u4
    (tests/cute_kernel/quantized_linear.py:494-517)."""

    def __init__(self, name: str, k: int, n: int, group_size: int, with_zp: bool = True):
        if k % group_size != 0:
            raise ValueError('k={} is not a multiple of the group size {}'.format(k, group_size))
        if n % 8 != 0:
            raise ValueError('n={} is not a multiple of 8'.format(n))
        self.name, self.k, self.n, self.group_size, self.with_zp = name, k, n, group_size, with_zp

    def __call__(self, a: torch.Tensor, b: torch.Tensor, scale: torch.Tensor, zeros: torch.Tensor = None) -> torch.Tensor:
        require_cuda(a, 'a')
        require_cuda(b, 'b')
        require_cuda(scale, 'scale')
        groups = self.k // self.group_size
        if a.dtype != torch.float16 or a.dim() != 2 or a.shape[1] != self.k:
            raise ValueError('expect float16 activations [M, {}], got {} {}'.format(self.k, a.dtype, list(a.shape)))
        if b.dim() != 2 or b.shape[0] != self.k or b.shape[1] * b.element_size() * 2 != self.n:
            raise ValueError('expect packed codes for a [{}, {}] weight, got {} {}'.format(self.k, self.n, b.dtype, list(b.shape)))
        if scale.dtype != torch.float16 or list(scale.shape) != [groups, self.n]:
            raise ValueError('expect float16 scales [{}, {}], got {} {}'.format(groups, self.n, scale.dtype, list(scale.shape)))
        zp = None
        if self.with_zp:
            if zeros is None or zeros.dtype != torch.float16 or list(zeros.shape) != [groups, self.n]:
                raise ValueError('expect float16 zero points [{}, {}]'.format(groups, self.n))
            require_cuda(zeros, 'zeros')
            zp = zeros.contiguous()
        a, b, scale = a.contiguous(), b.contiguous(), scale.contiguous()
        m = a.shape[0]
        c = torch.empty((m, self.n), dtype=torch.float16, device=a.device)
        with torch.cuda.device(a.device):
            ws_bytes = ffi.func('b200q_qlinear_f16_u4_workspace_bytes')(m, self.n, self.k, self.group_size)
            ws_ptr, ws_size = workspaces.get(a.device, ws_bytes)
            ffi.func('b200q_qlinear_f16_u4')(a.data_ptr(), b.data_ptr(), scale.data_ptr(), zp.data_ptr() if zp is not None else None,
                                            c.data_ptr(), m, self.n, self.k, self.group_size, ws_ptr, ws_size, current_stream_ptr(a.device))
        return c


def w4a16_linear(name: str, input_feats: int, output_feats: int, group_size: int, with_zp: bool = True) -> FpAIntBGemm:
    """tests/cute_kernel/quantized_linear.py:1103-1104."""
    return FpAIntBGemm(name, input_feats, output_feats, group_size, with_zp)
