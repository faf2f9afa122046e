"""Operator objects of the quantized path.

The reference represents every computation as an ``Operator(inputs, attributes, task)`` whose outputs
are produced when it is constructed on concrete tensors, and which graph passes re-create through
``reforward`` -- ``cls(*inputs, **attributes)``, so constructor keyword names must equal the attribute
keys (python/hidet/graph/operator.py:59-71,194-199).  These classes keep that contract (same class
names, same keyword names) on torch tensors; `run` calls libhidet_b200q.so through the host functions.
"""
from __future__ import annotations

from typing import Any, Dict, List, Union

import torch

from .. import quant


class Operator:
    """inputs + attributes -> outputs, computed on construction (the reference's imperative mode)."""

    def __init__(self, inputs: List[torch.Tensor], attributes: Dict[str, Any]):
        self.inputs = list(inputs)
        self.attrs = dict(attributes)
        self.outputs = self.run()

    @property
    def name(self) -> str:
        n = type(self).__name__
        return n[:-2] if n.endswith('Op') else n

    def run(self) -> List[torch.Tensor]:
        raise NotImplementedError

    def reforward(self, inputs: List[torch.Tensor], update_attributes: Dict[str, Any] = None) -> List[torch.Tensor]:
        attrs = dict(self.attrs)
        if update_attributes:
            attrs.update(update_attributes)
        return type(self)(*inputs, **attrs).outputs


class SymmetricQuantizationOp(Operator):
    """python/hidet/graph/ops/quant/symmetric.py:64-70"""

    def __init__(self, w: torch.Tensor, quant_type='int8', dims: Union[int, List[int]] = -1):
        super().__init__([w], {'dims': dims, 'quant_type': quant_type})

    def run(self):
        return list(quant.symmetric_quantize(self.inputs[0], self.attrs['quant_type'], dims=self.attrs['dims']))


class SymmetricDeQuantizationOp(Operator):
    """python/hidet/graph/ops/quant/symmetric.py:73-79"""

    def __init__(self, wq: torch.Tensor, scale: torch.Tensor, dims: Union[int, List[int]] = -1):
        super().__init__([wq, scale], {'dims': dims})

    def run(self):
        return [quant.symmetric_dequantize(self.inputs[0], self.inputs[1], dims=self.attrs['dims'])]


class SymmetricQuantizedMatmulOp(Operator):
    """python/hidet/graph/ops/quant/matmul.py:77-80"""

    def __init__(self, a: torch.Tensor, b: torch.Tensor, scale: torch.Tensor):
        super().__init__([a, b, scale], {})

    def run(self):
        from .transforms import resolve_operator

        resolved = resolve_operator(self)  # the resolve-variant step, applied eagerly
        if resolved is not None:
            return resolved
        return [quant.symmetric_quant_matmul(*self.inputs)]


class SymmetricQuantizedMatmulF16I8Op(Operator):
    """python/hidet/graph/ops/quant/matmul_f16_i8.py:488-498"""

    def __init__(self, a: torch.Tensor, b: torch.Tensor, scale: torch.Tensor, parallel_k_parts=1):
        if not (isinstance(parallel_k_parts, int) and not isinstance(parallel_k_parts, bool)):
            raise ValueError('parallel_k_parts must be an integer, got {}'.format(parallel_k_parts))
        super().__init__([a, b, scale], {'parallel_k_parts': parallel_k_parts})

    def run(self):
        return [quant.symmetric_quant_matmul_f16_i8(*self.inputs, parallel_k_parts=self.attrs['parallel_k_parts'])]
