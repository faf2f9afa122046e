"""The f16 x int8 quantized matmul on CUDA tensors.

Host-side mirror of python/hidet/graph/ops/quant/matmul.py:83-93,
python/hidet/graph/ops/quant/matmul_f16_i8.py:501-511 and
python/hidet/graph/ops/quant/matmul_f16_i8_atomic.py:555-565: same names, argument meaning, checks
and error messages; the kernels are those of libhidet_b200q.so.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import ffi
from ..runtime import current_stream_ptr, require_cuda, workspaces

_LAYOUTS = {'KN': ffi.LAYOUT_KN, 'NK': ffi.LAYOUT_NK}


def _check_operands(a: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, layout: str):
    require_cuda(a, 'a')
    require_cuda(weight, 'weight')
    require_cuda(scale, 'scale')
    if a.dim() < 2 or weight.dim() < 2:
        raise ValueError('a and b must have at least 2 dimensions, got shape {} and {}'.format(list(a.shape), list(weight.shape)))
    if a.shape[-1] % 2 != 0 or weight.shape[-1] % 2 != 0:
        raise ValueError('Expect the last dimension of the input tensors to be a multiple of 2')
    if a.dtype != torch.float16 or weight.dtype != torch.int8:
        raise ValueError('BatchMatmulF16Op only support float16, int8, got {} and {}'.format(a.dtype, weight.dtype))
    if weight.dim() != 2:
        raise ValueError('SymmetricQuantizedMatmul expect , got {} and {}'.format(list(a.shape), list(weight.shape)))
    if layout not in _LAYOUTS:
        raise ValueError("weight_layout must be 'KN' or 'NK', got {!r}".format(layout))
    k_w, n = (weight.shape[0], weight.shape[1]) if layout == 'KN' else (weight.shape[1], weight.shape[0])
    if a.shape[-1] != k_w:
        raise ValueError(
            'Matrix multiplication expect tensor A and B with shape [..., M, K] and [..., K, N], got {} and {}'.format(
                list(a.shape), list(weight.shape)))
    if scale.dtype != torch.float16:
        raise ValueError('Expect scale to be float16, got {}'.format(scale.dtype))
    if scale.dim() != 1 or scale.shape[0] != n:
        raise ValueError('Expect scale of shape [{}], got {}'.format(n, list(scale.shape)))
    if not (a.device == weight.device == scale.device):
        raise ValueError('a, weight and scale must be on one device')
    m = 1
    for d in a.shape[:-1]:
        m *= d
    return m, n, k_w


_ACTIVATIONS = {None: ffi.ACT_NONE, 'none': ffi.ACT_NONE, 'silu_mul': ffi.ACT_SILU_MUL}


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Two tensors of equal shape [..., F] -> [..., 2F] with gate[..., j] at column 2j and up[..., j] at 2j + 1:
    the column order activation='silu_mul' expects.  Works for the float weights before quantization, for
    int8 codes and for scales alike (quantization is per column, so it commutes with the interleaving)."""
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError('gate and up must have equal shapes and dtypes, got {} {} and {} {}'.format(list(gate.shape), gate.dtype, list(up.shape), up.dtype))
    return torch.stack((gate, up), dim=-1).reshape(*gate.shape[:-1], 2 * gate.shape[-1]).contiguous()


def symmetric_quant_matmul(a: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, weight_layout: str = 'KN',
                           out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                           residual: Optional[torch.Tensor] = None, activation: Optional[str] = None) -> torch.Tensor:
    """c[..., M, N] = a[..., M, K] @ (float16(weight) * scale), accumulated in fp32, rounded to f16 once.

    weight is int8 [K, N] with scale [N] (weight_layout='KN', the reference's contract,
    python/hidet/graph/ops/quant/matmul.py:30-32) or int8 [N, K] (weight_layout='NK', the layout
    torch.nn.Linear keeps; not offered by the reference).  `out`, if given, receives the result (a
    contiguous float16 CUDA tensor of the output shape), so that a caller replaying a fixed sequence
    of calls allocates nothing.

    bias [N], activation and residual are applied inside the kernel to the fp32 sums, in that order, and the
    result is rounded to f16 once -- what the reference gets by fusing the following element-wise operators
    into the matmul (python/hidet/graph/transforms/fuse_operator.py).  activation='silu_mul': the weight's
    columns are (gate_j, up_j) pairs (see interleave_gate_up) and the result, N / 2 wide, is
    silu(gate) * up.  residual has the shape of the result.
    """
    m, n, k = _check_operands(a, weight, scale, weight_layout)
    if activation not in _ACTIVATIONS:
        raise ValueError("activation must be None or 'silu_mul', got {!r}".format(activation))
    fused = bias is not None or residual is not None or _ACTIVATIONS[activation] != ffi.ACT_NONE
    n_out = n // 2 if _ACTIVATIONS[activation] == ffi.ACT_SILU_MUL else n
    a2 = a.contiguous()
    weight = weight.contiguous()
    scale = scale.contiguous()
    out_shape = list(a.shape[:-1]) + [n_out]
    if fused:
        if weight_layout != 'KN':
            raise ValueError("bias, residual and activation are fused for weight_layout='KN' only")
        if bias is not None:
            require_cuda(bias, 'bias')
            if bias.dtype != torch.float16 or list(bias.shape) != [n]:
                raise ValueError('Expect a float16 bias of shape [{}], got {} {}'.format(n, bias.dtype, list(bias.shape)))
            bias = bias.contiguous()
        if residual is not None:
            require_cuda(residual, 'residual')
            if residual.dtype != torch.float16 or list(residual.shape) != out_shape:
                raise ValueError('Expect a float16 residual of shape {}, got {} {}'.format(out_shape, residual.dtype, list(residual.shape)))
            residual = residual.contiguous()
    if out is None:
        c = torch.empty(out_shape, dtype=torch.float16, device=a.device)
    else:
        if list(out.shape) != out_shape or out.dtype != torch.float16 or out.device != a.device or not out.is_contiguous():
            raise ValueError('out must be a contiguous float16 tensor of shape {} on {}'.format(out_shape, a.device))
        c = out
    layout = _LAYOUTS[weight_layout]
    with torch.cuda.device(a.device):
        ws_bytes = ffi.func('b200q_qlinear_workspace_bytes')(m, n, k, layout)
        ws_ptr, ws_size = workspaces.get(a.device, ws_bytes)
        if fused:
            ep = ffi.Epilogue(bias.data_ptr() if bias is not None else None, residual.data_ptr() if residual is not None else None,
                              n_out, _ACTIVATIONS[activation])
            ffi.func('b200q_qlinear_f16_i8_fused')(
                a2.data_ptr(), weight.data_ptr(), scale.data_ptr(), c.data_ptr(), m, n, k, layout, ctypes.byref(ep), ws_ptr, ws_size,
                current_stream_ptr(a.device),
            )
        else:
            ffi.func('b200q_qlinear_f16_i8')(
                a2.data_ptr(), weight.data_ptr(), scale.data_ptr(), c.data_ptr(), m, n, k, layout, ws_ptr, ws_size,
                current_stream_ptr(a.device),
            )
    return c


def symmetric_quant_matmul_f16_i8(a: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, parallel_k_parts=1) -> torch.Tensor:
    """The reference's explicit split-K form: returns c[parallel_k_parts, ..., M, N]; the caller sums
    over the leading axis (python/hidet/graph/ops/quant/resolve.py:99)."""
    if not (isinstance(parallel_k_parts, int) and not isinstance(parallel_k_parts, bool)):
        raise ValueError('parallel_k_parts must be an integer, got {}'.format(parallel_k_parts))
    m, n, k = _check_operands(a, weight, scale, 'KN')
    if parallel_k_parts < 1:
        raise ValueError('parallel_k_parts must be positive, got {}'.format(parallel_k_parts))
    a2 = a.contiguous()
    weight = weight.contiguous()
    scale = scale.contiguous()
    c = torch.empty([parallel_k_parts] + list(a.shape[:-1]) + [n], dtype=torch.float16, device=a.device)
    with torch.cuda.device(a.device):
        ffi.func('b200q_qlinear_f16_i8_parts')(
            a2.data_ptr(), weight.data_ptr(), scale.data_ptr(), c.data_ptr(), m, n, k, parallel_k_parts,
            current_stream_ptr(a.device),
        )
    return c


def symmetric_quant_matmul_atomic_f16_i8(a: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, parallel_k_parts=1) -> torch.Tensor:
    """The reference's atomic split-K form returns the already summed c[..., M, N]
    (python/hidet/graph/ops/quant/matmul_f16_i8_atomic.py:31-86).  Here the split over K is chosen
    inside the library and summed in a fixed order, so `parallel_k_parts` is accepted and checked but
    does not change the result, which, unlike the reference's f16 atomics, is the same on every run."""
    if not (isinstance(parallel_k_parts, int) and not isinstance(parallel_k_parts, bool)):
        raise ValueError('parallel_k_parts must be an integer, got {}'.format(parallel_k_parts))
    return symmetric_quant_matmul(a, weight, scale)
