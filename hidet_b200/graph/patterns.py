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
from typing import Dict, List, Optional, Union

import torch
import torch.fx as fx
import torch.nn.functional as F

from .. import quant
from .operators import SymmetricDeQuantizationOp, SymmetricQuantizedMatmulOp
from .transforms import PURE_TARGETS, SubgraphRewriteRule, drop_unused_constants


def _fusable(k: int, n: int) -> bool:
    """The kernels with a fused epilogue take rows that are multiples of 16 bytes."""
    return n % 16 == 0 and k % 8 == 0


def quantized_linear_nk(a: torch.Tensor, wq_nk: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """The call made for a linear layer whose int8 weight was kept in torch's [N, K] layout."""
    return quant.symmetric_quant_matmul(a, wq_nk, scale, weight_layout='NK')


def quantized_matmul(a: torch.Tensor, wq: torch.Tensor, scale: torch.Tensor, bias: Optional[torch.Tensor] = None,
                     residual: Optional[torch.Tensor] = None, activation: Optional[str] = None) -> torch.Tensor:
    """The call the rewritten graph makes: the quantized matmul operator, resolved to the library kernel.
    With bias / residual / activation (folded in by QuantizedLinearEpilogueFusion) the kernel applies them
    itself; a residual that only broadcasts to the result is added afterwards."""
    if bias is None and residual is None and activation is None:
        return SymmetricQuantizedMatmulOp(a, wq, scale).outputs[0]
    n_out = wq.shape[1] // 2 if activation == 'silu_mul' else wq.shape[1]
    late = None
    if residual is not None and (list(residual.shape) != list(a.shape[:-1]) + [n_out] or residual.dtype != torch.float16):
        late, residual = residual, None
    out = quant.symmetric_quant_matmul(a, wq, scale, bias=bias, residual=residual, activation=activation)
    return out if late is None else out + late


_MATMULS = {torch.matmul, operator.matmul, torch.mm}
_LINEARS = {F.linear, torch._C._nn.linear}


def _eligible(w: torch.Tensor) -> bool:
    # the fused rule's conditions (linear.py:108-122): float16, 2-D, last dims even / multiple of 4
    return w.dtype == torch.float16 and w.dim() == 2 and w.is_cuda


class SymmetricLinearQuantizePattern(SubgraphRewriteRule):
    def __init__(self, quant_type: str = 'int8', dims: Union[int, List[int]] = 0, linear_weight_layout: str = 'KN'):
        """linear_weight_layout: what becomes of a torch.nn.Linear / F.linear weight W[N, K].  'KN' (default):
        transposed once at rewrite time into the reference's [K, N] layout, whose kernels take the fused
        epilogue.  'NK': kept as it is and quantized per row (dims=1) -- the same codes and scales -- and run
        by the [N, K] kernels; nothing is transposed, and the bias, if any, stays a separate add."""
        super().__init__('symmetric_linear_quantize')
        if quant_type != 'int8':
            raise ValueError('the fused quantized matmul takes int8 weights, got {}'.format(quant_type))
        if dims not in (0, [0]):
            raise ValueError('per-output-channel quantization of a [K, N] weight is dims=0, got {}'.format(dims))
        if linear_weight_layout not in ('KN', 'NK'):
            raise ValueError("linear_weight_layout must be 'KN' or 'NK', got {!r}".format(linear_weight_layout))
        self.quant_type = quant_type
        self.linear_weight_layout = linear_weight_layout

    def _install_nk(self, gm: fx.GraphModule, node: fx.Node, w_nk: torch.Tensor, idx: int):
        wq, scale = quant.symmetric_quantize(w_nk.contiguous(), self.quant_type, dims=-1)
        wq_name, scale_name = '_b200q_wq_{}'.format(idx), '_b200q_scale_{}'.format(idx)
        gm.register_buffer(wq_name, wq)
        gm.register_buffer(scale_name, scale)
        with gm.graph.inserting_before(node):
            return gm.graph.get_attr(wq_name), gm.graph.get_attr(scale_name)

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
                if self.linear_weight_layout == 'NK':
                    wq_node, scale_node = self._install_nk(gm, node, mod.weight.detach(), existing + count)
                    with gm.graph.inserting_before(node):
                        new = gm.graph.call_function(quantized_linear_nk, (node.args[0], wq_node, scale_node))
                        if mod.bias is not None:
                            bias_name = '_b200q_bias_{}'.format(existing + count)
                            gm.register_buffer(bias_name, mod.bias.detach())
                            new = gm.graph.call_function(torch.add, (new, gm.graph.get_attr(bias_name)))
                    node.replace_all_uses_with(new)
                    gm.graph.erase_node(node)
                    count += 1
                    continue
                wq_node, scale_node = self._install(gm, node, mod.weight.detach().t(), existing + count)
                with gm.graph.inserting_before(node):
                    if mod.bias is not None:
                        bias_name = '_b200q_bias_{}'.format(existing + count)
                        gm.register_buffer(bias_name, mod.bias.detach())
                        bias_node = gm.graph.get_attr(bias_name)
                        if _fusable(mod.weight.shape[1], mod.weight.shape[0]) and mod.bias.dtype == torch.float16:
                            new = gm.graph.call_function(quantized_matmul, (node.args[0], wq_node, scale_node), {'bias': bias_node})
                        else:
                            new = gm.graph.call_function(torch.add, (gm.graph.call_function(quantized_matmul, (node.args[0], wq_node, scale_node)), bias_node))
                    else:
                        new = gm.graph.call_function(quantized_matmul, (node.args[0], wq_node, scale_node))
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
                if self.linear_weight_layout == 'NK':
                    wq_node, scale_node = self._install_nk(gm, node, w_nk, existing + count)
                    with gm.graph.inserting_before(node):
                        new = gm.graph.call_function(quantized_linear_nk, (x, wq_node, scale_node))
                        if bias is not None:
                            new = gm.graph.call_function(torch.add, (new, bias))
                    node.replace_all_uses_with(new)
                    gm.graph.erase_node(node)
                    count += 1
                    continue
                wq_node, scale_node = self._install(gm, node, w_nk.t(), existing + count)
                with gm.graph.inserting_before(node):
                    bias_const = constants.get(bias.name) if isinstance(bias, fx.Node) else None
                    if bias is not None and bias_const is not None and bias_const.dtype == torch.float16 and _fusable(w_nk.shape[1], w_nk.shape[0]):
                        new = gm.graph.call_function(quantized_matmul, (x, wq_node, scale_node), {'bias': bias})
                    else:
                        new = gm.graph.call_function(quantized_matmul, (x, wq_node, scale_node))
                        if bias is not None:
                            new = gm.graph.call_function(torch.add, (new, bias))
                node.replace_all_uses_with(new)
                gm.graph.erase_node(node)
                count += 1
        return count


# The reference's name for the rule with the constant on the right (linear.py:25-49).
SymmetricLinearQuantizePatternR = SymmetricLinearQuantizePattern


def dequantized_weight(wq: torch.Tensor, scale: torch.Tensor, dims=0) -> torch.Tensor:
    """The call a two-step rewrite leaves in the graph: the dequantize operator."""
    return SymmetricDeQuantizationOp(wq, scale, dims=dims).outputs[0]


class SymmetricLinearQuantizePatternL(SubgraphRewriteRule):
    """matmul(W, x) with a constant 2-D float16 W[M, K] => matmul(dequant(wq, scale, dims), x)
    (python/hidet/graph/transforms/graph_patterns/quant/linear.py:52-84).  As in the reference, this
    form keeps a plain matmul behind a dequantize (its fused rule only matches the constant on the
    right, linear.py:87-124): the weight is stored in int8, the product is not fused."""

    def __init__(self, quant_type: str = 'int8', dims: Union[int, List[int]] = 0):
        super().__init__('symmetric_linear_quantize_left')
        self.quant_type = quant_type
        self.dims = dims

    def apply(self, gm: fx.GraphModule, constants: Dict[str, torch.Tensor]) -> int:
        count = 0
        existing = sum(1 for name, _ in gm.named_buffers() if name.startswith('_b200q_lwq_'))
        for node in list(gm.graph.nodes):
            if node.op != 'call_function' or node.target not in _MATMULS or len(node.args) != 2:
                continue
            w, x = node.args
            if not isinstance(w, fx.Node) or w.name not in constants or not _eligible(constants[w.name]):
                continue
            if isinstance(x, fx.Node) and x.name in constants:
                continue  # both constant: nothing to gain
            wq, scale = quant.symmetric_quantize(constants[w.name].contiguous(), self.quant_type, dims=self.dims)
            wq_name, scale_name = '_b200q_lwq_{}'.format(existing + count), '_b200q_lscale_{}'.format(existing + count)
            gm.register_buffer(wq_name, wq)
            gm.register_buffer(scale_name, scale)
            with gm.graph.inserting_before(node):
                wd = gm.graph.call_function(dequantized_weight, (gm.graph.get_attr(wq_name), gm.graph.get_attr(scale_name)), {'dims': self.dims})
                new = gm.graph.call_function(torch.matmul, (wd, x))
            node.replace_all_uses_with(new)
            gm.graph.erase_node(node)
            count += 1
        return count


class SymmetricQuantizeMatmulFused(SubgraphRewriteRule):
    """matmul(x, dequant(wq, scale, dims=0)) => symmetric_quant_matmul(x, wq, scale), under the conditions of
    python/hidet/graph/transforms/graph_patterns/quant/linear.py:87-124 (int8 2-D weight, per-column scale,
    last dimensions even / multiples of 4).  Serves graphs that were quantized in two steps."""

    def __init__(self):
        super().__init__('symmetric_quantize_matmul_fused')

    def apply(self, gm: fx.GraphModule, constants: Dict[str, torch.Tensor]) -> int:
        count = 0
        for node in list(gm.graph.nodes):
            if node.op != 'call_function' or node.target not in _MATMULS or len(node.args) != 2:
                continue
            x, wd = node.args
            if not isinstance(wd, fx.Node) or wd.op != 'call_function' or wd.target is not dequantized_weight:
                continue
            if wd.kwargs.get('dims', wd.args[2] if len(wd.args) > 2 else 0) not in (0, [0]):
                continue
            wq_node, scale_node = wd.args[0], wd.args[1]
            wq = constants.get(getattr(wq_node, 'name', None))
            scale = constants.get(getattr(scale_node, 'name', None))
            if wq is None or scale is None or wq.dtype != torch.int8 or wq.dim() != 2 or scale.dtype != torch.float16:
                continue
            if wq.shape[1] % 4 or wq.shape[0] % 2 or scale.shape[0] != wq.shape[1]:
                continue
            with gm.graph.inserting_before(node):
                new = gm.graph.call_function(quantized_matmul, (x, wq_node, scale_node))
            node.replace_all_uses_with(new)
            gm.graph.erase_node(node)
            count += 1
        return count


_SILUS = {F.silu, torch.nn.functional.silu}
_MULS = {operator.mul, torch.mul}
_ADDS = {operator.add, torch.add}


class QuantizedLinearEpilogueFusion(SubgraphRewriteRule):
    """Folds what follows a quantized linear into its kernel:
        silu(qmm(x, Wg)) * qmm(x, Wu)   =>  qmm(x, interleave(Wg, Wu), activation='silu_mul')   (SwiGLU; one launch, one pass over x)
        r + qmm(x, W)                   =>  qmm(x, W, residual=r)
    The reference gets there by fusing element-wise operators into the matmul task as prologues / epilogues
    (python/hidet/graph/transforms/fuse_operator.py, python/hidet/graph/ops/quant/matmul_f16_i8.py:95-99)."""

    def __init__(self):
        super().__init__('quantized_linear_epilogue_fusion')

    @staticmethod
    def _plain_qmm(node) -> bool:
        return isinstance(node, fx.Node) and node.op == 'call_function' and node.target is quantized_matmul and not node.kwargs and len(node.args) == 3

    def _is_silu(self, gm: fx.GraphModule, node) -> bool:
        if not isinstance(node, fx.Node):
            return False
        if node.op == 'call_function' and node.target in _SILUS:
            return len(node.args) == 1 and not node.kwargs.get('inplace', False)
        return node.op == 'call_module' and isinstance(gm.get_submodule(node.target), torch.nn.SiLU)

    def apply(self, gm: fx.GraphModule, constants: Dict[str, torch.Tensor]) -> int:
        count = 0
        buffers = dict(gm.named_buffers())

        def const_of(node):
            return buffers.get(node.target) if isinstance(node, fx.Node) and node.op == 'get_attr' else None

        existing = sum(1 for name in buffers if name.startswith('_b200q_gu_wq_'))
        for node in list(gm.graph.nodes):
            if node.op != 'call_function' or node.target not in _MULS or len(node.args) != 2:
                continue
            for act, up in (node.args, node.args[::-1]):
                if not (self._is_silu(gm, act) and self._plain_qmm(act.args[0]) and self._plain_qmm(up)):
                    continue
                gate = act.args[0]
                if gate.args[0] is not up.args[0] or len(gate.users) != 1 or len(act.users) != 1 or len(up.users) != 1:
                    continue
                wq_g, s_g, wq_u, s_u = (const_of(n) for n in (gate.args[1], gate.args[2], up.args[1], up.args[2]))
                if any(t is None for t in (wq_g, s_g, wq_u, s_u)) or wq_g.shape != wq_u.shape or not _fusable(wq_g.shape[0], 2 * wq_g.shape[1]):
                    continue
                wq_name, scale_name = '_b200q_gu_wq_{}'.format(existing + count), '_b200q_gu_scale_{}'.format(existing + count)
                gm.register_buffer(wq_name, quant.interleave_gate_up(wq_g, wq_u))
                gm.register_buffer(scale_name, quant.interleave_gate_up(s_g, s_u))
                with gm.graph.inserting_before(node):
                    new = gm.graph.call_function(quantized_matmul, (gate.args[0], gm.graph.get_attr(wq_name), gm.graph.get_attr(scale_name)),
                                                 {'activation': 'silu_mul'})
                node.replace_all_uses_with(new)
                for dead in (node, act, gate, up):
                    gm.graph.erase_node(dead)
                count += 1
                break
        for node in list(gm.graph.nodes):
            if node.op != 'call_function' or node.target not in _ADDS or len(node.args) != 2 or node.kwargs:
                continue
            for q, r in (node.args, node.args[::-1]):
                if not (isinstance(q, fx.Node) and q.op == 'call_function' and q.target is quantized_matmul and 'residual' not in q.kwargs):
                    continue
                if len(q.users) != 1 or not isinstance(r, fx.Node) or r is q:
                    continue
                wq = const_of(q.args[1])
                if wq is None or not _fusable(wq.shape[0], wq.shape[1]):
                    continue
                with gm.graph.inserting_before(node):
                    new = gm.graph.call_function(quantized_matmul, q.args, dict(q.kwargs, residual=r))
                node.replace_all_uses_with(new)
                gm.graph.erase_node(node)
                gm.graph.erase_node(q)
                count += 1
                break
        # weights that only the unfused calls used
        if count:
            drop_unused_constants(gm)
            used = {n.target for n in gm.graph.nodes if n.op == 'get_attr'}
            for name in list(buffers):
                if name.startswith('_b200q_') and name not in used and hasattr(gm, name):
                    delattr(gm, name)
        return count


class QuantizedLinearConcat(SubgraphRewriteRule):
    """Several plain quantized linears of the same input (the query / key / value projections of an attention block)
    become one with the weights side by side, and slices of its result:
        qmm(x, W1), qmm(x, W2), ...   =>   y = qmm(x, [W1 | W2 | ...]);  y[..., 0:n1], y[..., n1:n1+n2], ...
    One launch and one pass over x instead of several; per-column scales make the concatenation exact.  The
    reference has this rewrite for float16 matmuls only (python/hidet/graph/transforms/graph_patterns/matmul_patterns.py).
    Runs after the epilogue fusion, which takes the gate / up pairs and the linears with a residual."""

    def __init__(self):
        super().__init__('quantized_linear_concat')

    def apply(self, gm: fx.GraphModule, constants: Dict[str, torch.Tensor]) -> int:
        buffers = dict(gm.named_buffers())

        def const_of(node):
            return buffers.get(node.target) if isinstance(node, fx.Node) and node.op == 'get_attr' else None

        groups: Dict[fx.Node, List[fx.Node]] = {}
        for node in gm.graph.nodes:
            if QuantizedLinearEpilogueFusion._plain_qmm(node) and isinstance(node.args[0], fx.Node):
                wq, scale = const_of(node.args[1]), const_of(node.args[2])
                if wq is not None and scale is not None and wq.dim() == 2 and wq.dtype == torch.int8:
                    groups.setdefault(node.args[0], []).append(node)
        existing = sum(1 for name in buffers if name.startswith('_b200q_cat_wq_'))
        count = 0
        for x, members in groups.items():
            if len(members) < 2:
                continue
            weights = [const_of(n.args[1]) for n in members]
            scales = [const_of(n.args[2]) for n in members]
            k = weights[0].shape[0]
            if any(w.shape[0] != k or w.shape[1] % 8 for w in weights) or any(sc.dtype != scales[0].dtype for sc in scales):
                continue
            if not _fusable(k, sum(w.shape[1] for w in weights)):
                continue
            wq_name, scale_name = '_b200q_cat_wq_{}'.format(existing + count), '_b200q_cat_scale_{}'.format(existing + count)
            gm.register_buffer(wq_name, torch.cat(weights, dim=1).contiguous())
            gm.register_buffer(scale_name, torch.cat(scales, dim=0).contiguous())
            with gm.graph.inserting_before(members[0]):   # every member depends on x and constants only
                merged = gm.graph.call_function(quantized_matmul, (x, gm.graph.get_attr(wq_name), gm.graph.get_attr(scale_name)))
                begin = 0
                for member, w in zip(members, weights):
                    piece = gm.graph.call_function(operator.getitem, (merged, (Ellipsis, slice(begin, begin + w.shape[1]))))
                    member.replace_all_uses_with(piece)
                    begin += w.shape[1]
            for member in members:
                gm.graph.erase_node(member)
            count += 1
        if count:
            drop_unused_constants(gm)
            used = {n.target for n in gm.graph.nodes if n.op == 'get_attr'}
            for name in list(buffers):
                if name.startswith('_b200q_') and name not in used and hasattr(gm, name):
                    delattr(gm, name)
        return count


def quantized_embedding(indices: torch.Tensor, wq: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """The call the rewritten graph makes for an embedding: lookup in the row-quantized table."""
    return quant.symmetric_dequantize_take(wq, scale, indices)


class SymmetricEmbeddingQuantizePattern(SubgraphRewriteRule):
    """embedding(W, ind) with a constant 2-D table => lookup in the table quantized per row
    (python/hidet/graph/transforms/graph_patterns/quant/embedding.py:22-39: take(dequant(wq, scale, dims=-1),
    ind, axis=0), here as one kernel).  Matches torch.nn.Embedding leaf modules and F.embedding calls with
    int32 / int64 indices and no padding / max-norm options."""

    def __init__(self, quant_type: str = 'int8'):
        super().__init__('symmetric_embedding_quantize')
        self.quant_type = quant_type

    def _install(self, gm: fx.GraphModule, node: fx.Node, table: torch.Tensor, idx: int):
        wq, scale = quant.symmetric_quantize(table.contiguous(), self.quant_type, dims=-1)
        wq_name, scale_name = '_b200q_emb_wq_{}'.format(idx), '_b200q_emb_scale_{}'.format(idx)
        gm.register_buffer(wq_name, wq)
        gm.register_buffer(scale_name, scale)
        with gm.graph.inserting_before(node):
            return gm.graph.get_attr(wq_name), gm.graph.get_attr(scale_name)

    def apply(self, gm: fx.GraphModule, constants: Dict[str, torch.Tensor]) -> int:
        count = 0
        existing = sum(1 for name, _ in gm.named_buffers() if name.startswith('_b200q_emb_wq_'))
        for node in list(gm.graph.nodes):
            table, ind = None, None
            if node.op == 'call_module':
                mod = gm.get_submodule(node.target)
                if isinstance(mod, torch.nn.Embedding) and mod.max_norm is None and not mod.sparse and len(node.args) == 1:
                    table, ind = mod.weight.detach(), node.args[0]
            elif node.op == 'call_function' and node.target is F.embedding:
                w = node.args[1] if len(node.args) > 1 else node.kwargs.get('weight')
                # padding_idx, max_norm, norm_type, scale_grad_by_freq, sparse: only their defaults (a padding index
                # changes nothing in the forward pass either)
                extras = list(node.args[2:]) + [node.kwargs.get(k) for k in ('max_norm', 'norm_type', 'scale_grad_by_freq', 'sparse')]
                plain = all(v in (None, False, 2.0, -1) or (i == 0 and isinstance(v, int)) for i, v in enumerate(extras))
                if len(node.args) > 3 and node.args[3] is not None:
                    plain = False  # max_norm renormalises the table
                if isinstance(w, fx.Node) and w.name in constants and plain:
                    table, ind = constants[w.name], node.args[0]
            if table is None or table.dim() != 2 or not table.is_cuda or table.dtype not in (torch.float16, torch.bfloat16, torch.float32):
                continue
            wq_node, scale_node = self._install(gm, node, table, existing + count)
            with gm.graph.inserting_before(node):
                new = gm.graph.call_function(quantized_embedding, (ind, wq_node, scale_node))
            node.replace_all_uses_with(new)
            gm.graph.erase_node(node)
            count += 1
        return count


PURE_TARGETS.update({quantized_linear_nk, quantized_matmul, dequantized_weight, quantized_embedding})


def symmetric_linear_patterns(quant_type: str = 'int8', dims: Union[int, List[int]] = 0) -> List[SubgraphRewriteRule]:
    """python/hidet/graph/transforms/graph_patterns/quant/__init__.py:31-46 and linear.py:87-92: the rule for
    the constant on the right, the rule for the constant on the left, and the fusion of a two-step graph."""
    return [SymmetricLinearQuantizePatternR(quant_type=quant_type, dims=dims), SymmetricLinearQuantizePatternL(quant_type=quant_type, dims=dims),
            SymmetricQuantizeMatmulFused()]


def symmetric_embedding_quantize_patterns(quant_type: str = 'int8') -> List[SubgraphRewriteRule]:
    """python/hidet/graph/transforms/graph_patterns/quant/embedding.py:42-43"""
    return [SymmetricEmbeddingQuantizePattern(quant_type=quant_type)]


def default_patterns() -> List[SubgraphRewriteRule]:
    """python/hidet/graph/transforms/graph_patterns/quant/__init__.py:19-28: embedding tables and linear layers; then
    the fusion of what follows a quantized linear into its kernel (in the reference a later pass, fuse_operator), then
    the merging of the quantized linears that are left sharing an input."""
    return (symmetric_embedding_quantize_patterns(quant_type='int8') + symmetric_linear_patterns(quant_type='int8', dims=0) +
            [QuantizedLinearEpilogueFusion(), QuantizedLinearConcat()])
