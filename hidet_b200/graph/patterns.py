"""Rewrite rules that quantize linear layers of an fx graph.

Counterparts of SymmetricLinearQuantizePatternR / SymmetricQuantizeMatmulFused
(python/hidet/graph/transforms/graph_patterns/quant/linear.py:25-129): ``matmul(x, W)`` with a constant
2-D float16 ``W[K, N]`` becomes ``symmetric_quant_matmul(x, wq, scale)`` with ``wq, scale =
symmetric_quantize(W, dims=0)`` computed once, when the rule fires.  The reference builds this in two
steps (dequantize pattern, then fusion); with a prebuilt fused kernel the intermediate form has no use.

``linear(x, W[N, K], b)`` -- what torch.nn.Linear traces to, and what the reference's patterns do not
handle (they rebuild a plain matmul, python/hidet/graph/transforms/graph_patterns/quant/linear.py:37-49) --
is quantized per output channel as well: the constant is transposed once to [K, N] at rewrite time,
which gives the same codes and scales as quantizing W[N, K] over dims=1, and the bias add stays.
"""
from __future__ import annotations

import operator
from typing import Dict, List, Union

import torch
import torch.fx as fx
import torch.nn.functional as F

from .. import quant
from .operators import SymmetricQuantizedMatmulOp
from .transforms import SubgraphRewriteRule


def quantized_matmul(a: torch.Tensor, wq: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """The call the rewritten graph makes: the quantized matmul operator, resolved to the library kernel."""
    return SymmetricQuantizedMatmulOp(a, wq, scale).outputs[0]


_MATMULS = {torch.matmul, operator.matmul, torch.mm}
_LINEARS = {F.linear, torch._C._nn.linear}


def _eligible(w: torch.Tensor) -> bool:
    # the fused rule's conditions (linear.py:108-122): float16, 2-D, last dims even / multiple of 4
    return w.dtype == torch.float16 and w.dim() == 2 and w.is_cuda


class SymmetricLinearQuantizePattern(SubgraphRewriteRule):
    def __init__(self, quant_type: str = 'int8', dims: Union[int, List[int]] = 0):
        super().__init__('symmetric_linear_quantize')
        if quant_type != 'int8':
            raise ValueError('the fused quantized matmul takes int8 weights, got {}'.format(quant_type))
        if dims not in (0, [0]):
            raise ValueError('per-output-channel quantization of a [K, N] weight is dims=0, got {}'.format(dims))
        self.quant_type = quant_type

    def _install(self, gm: fx.GraphModule, node: fx.Node, w_kn: torch.Tensor, idx: int):
        wq, scale = quant.symmetric_quantize(w_kn.contiguous(), self.quant_type, dims=0)
        wq_name, scale_name = '_b200q_wq_{}'.format(idx), '_b200q_scale_{}'.format(idx)
        gm.register_buffer(wq_name, wq)
        gm.register_buffer(scale_name, scale)
        with gm.graph.inserting_before(node):
            wq_node = gm.graph.get_attr(wq_name)
            scale_node = gm.graph.get_attr(scale_name)
        return wq_node, scale_node

    def apply(self, gm: fx.GraphModule, constants: Dict[str, torch.Tensor]) -> int:
        count = 0
        existing = sum(1 for name, _ in gm.named_buffers() if name.startswith('_b200q_wq_'))
        for node in list(gm.graph.nodes):
            if node.op == 'call_module':
                # a torch.nn.Linear kept as a leaf module (fx.symbolic_trace does that)
                mod = gm.get_submodule(node.target)
                if not isinstance(mod, torch.nn.Linear) or not _eligible(mod.weight) or len(node.args) != 1:
                    continue
                if mod.weight.shape[1] % 2 or mod.weight.shape[0] % 4:
                    continue
                wq_node, scale_node = self._install(gm, node, mod.weight.detach().t(), existing + count)
                with gm.graph.inserting_before(node):
                    new = gm.graph.call_function(quantized_matmul, (node.args[0], wq_node, scale_node))
                    if mod.bias is not None:
                        bias_name = '_b200q_bias_{}'.format(existing + count)
                        gm.register_buffer(bias_name, mod.bias.detach())
                        new = gm.graph.call_function(torch.add, (new, gm.graph.get_attr(bias_name)))
                node.replace_all_uses_with(new)
                gm.graph.erase_node(node)
                count += 1
                continue
            if node.op != 'call_function':
                continue
            if node.target in _MATMULS and len(node.args) == 2:
                x, w = node.args
                if not isinstance(w, fx.Node) or w.name not in constants or not _eligible(constants[w.name]):
                    continue
                w_kn = constants[w.name]
                if w_kn.shape[0] % 2 or w_kn.shape[1] % 4:
                    continue
                wq_node, scale_node = self._install(gm, node, w_kn, existing + count)
                with gm.graph.inserting_before(node):
                    new = gm.graph.call_function(quantized_matmul, (x, wq_node, scale_node))
                node.replace_all_uses_with(new)
                gm.graph.erase_node(node)
                count += 1
            elif node.target in _LINEARS:
                x, w = node.args[0], node.args[1]
                bias = node.args[2] if len(node.args) > 2 else node.kwargs.get('bias')
                if not isinstance(w, fx.Node) or w.name not in constants or not _eligible(constants[w.name]):
                    continue
                w_nk = constants[w.name]
                if w_nk.shape[1] % 2 or w_nk.shape[0] % 4:
                    continue
                wq_node, scale_node = self._install(gm, node, w_nk.t(), existing + count)
                with gm.graph.inserting_before(node):
                    new = gm.graph.call_function(quantized_matmul, (x, wq_node, scale_node))
                    if bias is not None:
                        new = gm.graph.call_function(torch.add, (new, bias))
                node.replace_all_uses_with(new)
                gm.graph.erase_node(node)
                count += 1
        return count


def symmetric_linear_patterns(quant_type: str = 'int8', dims: Union[int, List[int]] = 0) -> List[SubgraphRewriteRule]:
    """python/hidet/graph/transforms/graph_patterns/quant/__init__.py:31-46"""
    return [SymmetricLinearQuantizePattern(quant_type=quant_type, dims=dims)]


def default_patterns() -> List[SubgraphRewriteRule]:
    """python/hidet/graph/transforms/graph_patterns/quant/__init__.py:19-28 (the embedding rule of the
    reference is outside this path)."""
    return symmetric_linear_patterns(quant_type='int8', dims=0)
