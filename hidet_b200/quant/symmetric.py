"""symmetric_quantize / symmetric_dequantize on CUDA tensors.

Host-side mirror of python/hidet/graph/ops/quant/symmetric.py:82-88: same function names, argument
names, defaults and output shapes; the kernels are those of libhidet_b200q.so.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple, Union

import torch

from .. import ffi
from ..runtime import FLOAT_CODES, QUANT_CODES, QUANT_NAMES, current_stream_ptr, require_cuda


def _normalize_dims(dims: Union[int, Sequence[int]], rank: int) -> List[int]:
    """Same normalisation as hidet.graph.ops.utils.normalize_dim: negative dims count from the end."""
    if isinstance(dims, int):
        dims = [dims]
    out = []
    for d in dims:
        if not -rank <= d < rank:
            raise ValueError('dim {} is out of range for a tensor of rank {}'.format(d, rank))
        out.append(d % rank)
    if len(set(out)) != len(out):
        raise ValueError('duplicate dims: {}'.format(list(dims)))
    return sorted(out)


def _as_2d(shape: Sequence[int], dims: List[int]) -> Tuple[int, int, int, List[int]]:
    """View a tensor of `shape`, reduced over `dims`, as [rows, cols] reduced over one of the two.

    Returns (rows, cols, reduce_dim, scale_shape).  The reduced dims must be a prefix or a suffix of
    the shape, which covers every use in the reference (dims=0 and dims=-1 of 2-D weights).
    """
    rank = len(shape)
    keep = [i for i in range(rank) if i not in dims]
    scale_shape = [shape[i] for i in keep]
    numel_red = 1
    for i in dims:
        numel_red *= shape[i]
    numel_keep = 1
    for i in keep:
        numel_keep *= shape[i]
    if dims == list(range(rank - len(dims), rank)):  # suffix: [keep..., reduced...]
        return numel_keep, numel_red, 1, scale_shape
    if dims == list(range(len(dims))):  # prefix: [reduced..., keep...]
        return numel_red, numel_keep, 0, scale_shape
    raise NotImplementedError(
        'symmetric quantization over dims {} of a rank-{} tensor: only leading or trailing dims are supported'.format(dims, rank)
    )


def _quant_dtype(quant_type) -> torch.dtype:
    if isinstance(quant_type, torch.dtype):
        dt = quant_type
    else:
        name = getattr(quant_type, 'name', quant_type)  # also accepts a hidet DataType
        if name not in QUANT_NAMES:
            raise ValueError('unsupported quant_type {!r}: expected int8 or int16'.format(quant_type))
        dt = QUANT_NAMES[name]
    if dt not in QUANT_CODES:
        raise ValueError('unsupported quant_type {!r}: expected int8 or int16'.format(quant_type))
    return dt


def symmetric_quantize(w: torch.Tensor, quant_type: Union[str, torch.dtype] = 'int8', dims: Union[int, List[int]] = -1):
    """Returns (wq, scale): scale = max|w| over `dims` / qmax, wq = quant_type(round(w / scale)).

    wq has w's shape; scale has w's dtype and w's shape without `dims`.  Bit-identical to the
    reference's result for the same input (python/hidet/graph/ops/quant/symmetric.py:23-47).
    """
    require_cuda(w, 'w')
    if w.dtype not in FLOAT_CODES:
        raise ValueError('symmetric_quantize expects float16, bfloat16 or float32, got {}'.format(w.dtype))
    qdtype = _quant_dtype(quant_type)
    dims_n = _normalize_dims(dims, w.dim())
    rows, cols, reduce_dim, scale_shape = _as_2d(list(w.shape), dims_n)
    w = w.contiguous()
    wq = torch.empty(w.shape, dtype=qdtype, device=w.device)
    scale = torch.empty(scale_shape, dtype=w.dtype, device=w.device)
    with torch.cuda.device(w.device):
        ffi.func('b200q_symmetric_quantize')(
            w.data_ptr(), wq.data_ptr(), scale.data_ptr(), rows, cols, FLOAT_CODES[w.dtype], QUANT_CODES[qdtype], reduce_dim,
            current_stream_ptr(w.device),
        )
    return wq, scale


def symmetric_dequantize(wq: torch.Tensor, scale: torch.Tensor, dims: Union[int, List[int]] = -1) -> torch.Tensor:
    """Returns scale.dtype(wq) * scale, scale broadcast along `dims`
    (python/hidet/graph/ops/quant/symmetric.py:50-61)."""
    require_cuda(wq, 'wq')
    require_cuda(scale, 'scale')
    if wq.dtype not in QUANT_CODES:
        raise ValueError('symmetric_dequantize expects int8 or int16 values, got {}'.format(wq.dtype))
    if scale.dtype not in FLOAT_CODES:
        raise ValueError('symmetric_dequantize expects a float16, bfloat16 or float32 scale, got {}'.format(scale.dtype))
    dims_n = _normalize_dims(dims, wq.dim())
    rows, cols, reduce_dim, scale_shape = _as_2d(list(wq.shape), dims_n)
    if list(scale.shape) != scale_shape:
        raise ValueError('scale has shape {}, expected {} for wq of shape {} and dims {}'.format(
            list(scale.shape), scale_shape, list(wq.shape), dims))
    wq = wq.contiguous()
    scale = scale.contiguous()
    w = torch.empty(wq.shape, dtype=scale.dtype, device=wq.device)
    with torch.cuda.device(wq.device):
        ffi.func('b200q_symmetric_dequantize')(
            wq.data_ptr(), scale.data_ptr(), w.data_ptr(), rows, cols, FLOAT_CODES[scale.dtype], QUANT_CODES[wq.dtype], reduce_dim,
            current_stream_ptr(wq.device),
        )
    return w


def symmetric_dequantize_take(wq: torch.Tensor, scale: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """take(symmetric_dequantize(wq, scale, dims=-1), indices, axis=0) in one kernel: the lookup the
    reference's embedding rule leaves in the graph (python/hidet/graph/transforms/graph_patterns/quant/
    embedding.py:22-39), without materialising the dequantized table.  wq is int8 / int16 [vocab, dim]
    quantized per row, scale [vocab]; indices are int32 or int64 of any shape; the result has shape
    indices.shape + [dim] and scale's dtype, and equals the rows of the dequantized table bit for bit."""
    require_cuda(wq, 'wq')
    require_cuda(scale, 'scale')
    require_cuda(indices, 'indices')
    if wq.dim() != 2 or wq.dtype not in QUANT_CODES:
        raise ValueError('expect a 2-D int8 or int16 table, got {} of shape {}'.format(wq.dtype, list(wq.shape)))
    if scale.dtype not in FLOAT_CODES or list(scale.shape) != [wq.shape[0]]:
        raise ValueError('scale has shape {}, expected [{}] (one scale per table row)'.format(list(scale.shape), wq.shape[0]))
    if indices.dtype not in (torch.int32, torch.int64):
        raise ValueError('indices must be int32 or int64, got {}'.format(indices.dtype))
    wq = wq.contiguous()
    scale = scale.contiguous()
    idx = indices.contiguous()
    out = torch.empty(list(indices.shape) + [wq.shape[1]], dtype=scale.dtype, device=wq.device)
    with torch.cuda.device(wq.device):
        ffi.func('b200q_embedding_dequantize')(
            wq.data_ptr(), scale.data_ptr(), idx.data_ptr(), out.data_ptr(), wq.shape[0], wq.shape[1], idx.numel(),
            FLOAT_CODES[scale.dtype], QUANT_CODES[wq.dtype], idx.element_size(), current_stream_ptr(wq.device),
        )
    return out
