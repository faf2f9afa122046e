"""Device plumbing for the host layer: dtype codes, pointers, streams and the scratch workspace.

torch is used for device memory and streams only; every computation happens inside
libhidet_b200q.so.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from . import ffi

FLOAT_CODES = {torch.float16: ffi.F16, torch.bfloat16: ffi.BF16, torch.float32: ffi.F32}
QUANT_CODES = {torch.int8: ffi.I8, torch.int16: ffi.I16}
QUANT_NAMES = {'int8': torch.int8, 'i8': torch.int8, 'int16': torch.int16, 'i16': torch.int16}


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError('{} must be a torch.Tensor, got {}'.format(name, type(t).__name__))
    if not t.is_cuda:
        raise ffi.BackendException(
            '{} lives on {}: hidet_b200 runs on CUDA devices only and has no CPU implementation'.format(name, t.device)
        )


def current_stream_ptr(device: torch.device) -> int:
    """The stream kernels are launched on: torch's current stream, as in the reference, whose runtime
    asks torch for it through a callback (src/hidet/runtime/cuda/context.cpp:78-88)."""
    return torch.cuda.current_stream(device).cuda_stream


class _Workspaces:
    """Grow-only, zero-initialised scratch per (device, stream), the role request_cuda_workspace
    plays in the reference (src/hidet/runtime/cuda/context.cpp:31-49,90-104).  The library keeps the
    part that must be zero (its tile counters) zero between calls, so a buffer is cleared only when it
    is created."""

    def __init__(self):
        self._buffers: Dict[Tuple[int, int], torch.Tensor] = {}

    def get(self, device: torch.device, nbytes: int) -> Tuple[int, int]:
        if nbytes == 0:
            return 0, 0
        index = device.index if device.index is not None else torch.cuda.current_device()
        key = (index, current_stream_ptr(device))
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < nbytes:
            size = 1 << max(20, (nbytes - 1).bit_length())
            buf = torch.zeros(size, dtype=torch.uint8, device=torch.device('cuda', index))
            self._buffers[key] = buf
        return buf.data_ptr(), buf.numel()

    def clear(self) -> None:
        self._buffers.clear()


workspaces = _Workspaces()
