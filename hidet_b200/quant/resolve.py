"""Split-K choice and the resolve rule of the quantized matmul.

Mirror of python/hidet/graph/ops/quant/resolve.py:23-100.  The reference rewrites
``symmetric_quant_matmul(a, b, scale)`` into ``symmetric_quant_matmul_f16_i8(a, b, scale, k_parts).sum(0)``
with ``k_parts`` taken from ``hidet.option.parallel_k``.  Here the split over K is chosen inside the
library and summed in the kernel, so the rule resolves to one fused call; ``resolve_k_parts`` keeps the
reference's arithmetic for callers that ask for the explicit form.
"""
from __future__ import annotations

from typing import Sequence, Union


def cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def resolve_k_parts(a_shape: Sequence[int], b_shape: Sequence[int], parallel_k: Union[str, int] = 'disabled') -> int:
    """The reference's k_parts for a[..., M, K] x b[K, N] (python/hidet/graph/ops/quant/resolve.py:42-96).

    'disabled' -> 1 (the reference's default, python/hidet/option.py:366)
    'default'  -> min(ceil(400 / (batch * ceil(M/64) * ceil(N/64))), ceil(K/64))
    int        -> clamped to 1..32
    'search'   -> the reference times ten candidates; there is nothing to search here (one kernel
                  handles the split), so this answers like 'default'.
    """
    m, k = a_shape[-2], a_shape[-1]
    n = b_shape[-1]
    batch = 1
    for d in a_shape[:-2]:
        batch *= d
    if isinstance(parallel_k, bool):
        raise ValueError('invalid parallel_k: {}'.format(parallel_k))
    if isinstance(parallel_k, int):
        return min(max(parallel_k, 1), 32)
    if parallel_k == 'disabled':
        return 1
    if parallel_k in ('default', 'search'):
        estimate_blocks = batch * cdiv(m, 64) * cdiv(n, 64)
        estimate_concurrent_blocks = 80 * 5
        max_k_parts = cdiv(k, 64)
        return min(cdiv(estimate_concurrent_blocks, estimate_blocks), max_k_parts)
    raise ValueError('invalid parallel_k: {}'.format(parallel_k))
