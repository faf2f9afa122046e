"""Capture and replay of a sequence of launches as one CUDA graph.

Mirror of hidet.cuda.graph.CudaGraph (python/hidet/cuda/graph.py:88-200): the graph is built from a
function that creates the (static) input tensors and a function that runs the launches on them;
``run_async(inputs)`` copies new inputs into the static ones and replays; the outputs are static
tensors that each replay overwrites.  The reference uses this for its 'reduce-overhead' mode
(python/hidet/graph/frontend/torch/dynamo_backends.py:38-52); for the quantized linear it removes the
per-call host work, which at decode sizes costs more than the kernels themselves.

Capture and replay are torch.cuda.CUDAGraph; every launch of libhidet_b200q.so is capturable (no
allocation, no synchronisation; tensor maps travel as kernel parameters).
"""
from __future__ import annotations

from typing import Any, Callable, List, Optional, Sequence

import torch


class CudaGraph:
    def __init__(self, f_create_inputs: Callable[[], List[torch.Tensor]], f_run: Callable[[List[torch.Tensor]], List[torch.Tensor]],
                 ref_objs: Optional[Sequence[Any]] = None, num_warmup: int = 2):
        self._ref_objs = list(ref_objs) if ref_objs is not None else []
        self._inputs: List[torch.Tensor] = list(f_create_inputs())
        if not self._inputs or not all(t.is_cuda for t in self._inputs):
            raise ValueError('f_create_inputs must return CUDA tensors')
        device = self._inputs[0].device
        self._stream = torch.cuda.Stream(device)
        self._stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(self._stream):
            for _ in range(max(num_warmup, 1)):  # allocates per-stream workspaces before the capture
                f_run(self._inputs)
            self._stream.synchronize()
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph, stream=self._stream):
                outputs = f_run(self._inputs)
        self._outputs: List[torch.Tensor] = list(outputs) if isinstance(outputs, (list, tuple)) else [outputs]

    @property
    def inputs(self) -> List[torch.Tensor]:
        return self._inputs

    @property
    def outputs(self) -> List[torch.Tensor]:
        return self._outputs

    def copy_inputs(self, inputs: Optional[Sequence[torch.Tensor]], stream: torch.cuda.Stream) -> None:
        if inputs is None:
            return
        if len(inputs) != len(self._inputs):
            raise ValueError('expect {} inputs, got {}'.format(len(self._inputs), len(inputs)))
        with torch.cuda.stream(stream):
            for dst, src in zip(self._inputs, inputs):
                if src is not dst:
                    dst.copy_(src, non_blocking=True)

    def run_async(self, inputs: Optional[Sequence[torch.Tensor]] = None, stream: Optional[torch.cuda.Stream] = None) -> List[torch.Tensor]:
        """Copy `inputs` (device or pinned host tensors) into the static inputs, replay, return the static
        outputs; everything is ordered on `stream` (default: the current stream) and nothing is waited for."""
        stream = stream if stream is not None else torch.cuda.current_stream(self._inputs[0].device)
        self.copy_inputs(inputs, stream)
        with torch.cuda.stream(stream):
            self._graph.replay()
        return self._outputs

    def __call__(self, *inputs: torch.Tensor):
        outputs = self.run(inputs if inputs else None)
        return outputs[0] if len(outputs) == 1 else outputs

    def run(self, inputs: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
        outputs = self.run_async(inputs)
        torch.cuda.current_stream(self._inputs[0].device).synchronize()
        return outputs
