"""Pass context, resolve rules and the quantization pass over torch.fx graphs.

Mirrors, for the quantized-linear path only:
  * PassContext.set_precision('int8') / add_quantize_rules (python/hidet/graph/transforms/base.py:112-165)
  * register_resolve_rule / ResolveRule (python/hidet/graph/transforms/resolve_variant.py:27-62)
  * the selective-quantize pass (python/hidet/graph/transforms/selective_quantize.py:20-28) and the
    rewrite rules it applies (python/hidet/graph/transforms/graph_patterns/quant/linear.py:25-129)

The reference rewrites its own FlowGraph; here the graph is a torch.fx.GraphModule (what torch.compile
hands to a backend), and a "constant weight" is a parameter or buffer of that module, or a
placeholder bound to a parameter at compile time.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Type

import torch
import torch.fx as fx

from .. import quant
from ..quant.resolve import resolve_k_parts
from .operators import Operator, SymmetricQuantizedMatmulOp


# ---------------------------------------------------------------------------------------------
# resolve rules
# ---------------------------------------------------------------------------------------------
class ResolveRule:
    """Replaces an operator by a variant; return None to leave it (resolve_variant.py:27-53)."""

    def resolve(self, op: Operator) -> Optional[List[torch.Tensor]]:
        raise NotImplementedError


_resolve_rules: Dict[Type[Operator], List[ResolveRule]] = {}


def register_resolve_rule(op_cls: Type[Operator]):
    """Decorator; rules registered later are tried first, as in the reference (resolve_variant.py:56-62)."""

    def wrapper(rule_cls: Type[ResolveRule]):
        _resolve_rules.setdefault(op_cls, []).append(rule_cls())
        return rule_cls

    return wrapper


def resolve_operator(op: Operator) -> Optional[List[torch.Tensor]]:
    for rule in reversed(_resolve_rules.get(type(op), [])):
        out = rule.resolve(op)
        if out is not None:
            return out
    return None


@register_resolve_rule(SymmetricQuantizedMatmulOp)
class QuantSymmetricResolveRule(ResolveRule):
    """The reference rule turns the op into symmetric_quant_matmul_f16_i8(a, b, scale, k_parts).sum(0)
    (python/hidet/graph/ops/quant/resolve.py:23-100).  The library's kernels split K themselves and sum
    in the kernel, so the variant is one fused call; k_parts computed the reference's way is kept on
    the rule for inspection only."""

    parallel_k = 'disabled'

    def resolve(self, op: Operator) -> Optional[List[torch.Tensor]]:
        a, b, scale = op.inputs
        if not a.is_cuda or torch.cuda.get_device_capability(a.device) < (8, 0):
            return None
        self.last_k_parts = resolve_k_parts(list(a.shape), list(b.shape), self.parallel_k)
        return [quant.symmetric_quant_matmul(a, b, scale)]


# ---------------------------------------------------------------------------------------------
# pass context
# ---------------------------------------------------------------------------------------------
class SubgraphRewriteRule:
    """One rewrite over an fx graph.  `apply` returns the number of rewrites it made."""

    def __init__(self, name: str = ''):
        self.name = name or type(self).__name__

    def apply(self, gm: fx.GraphModule, constants: Dict[str, torch.Tensor]) -> int:
        raise NotImplementedError


class PassContext:
    """with PassContext() as ctx: ctx.set_precision('int8'); optimize(gm)"""

    _stack: List['PassContext'] = []

    def __init__(self):
        self.configs: Dict[str, Any] = {'precision': None, 'quantize_patterns': [], 'verbose': False}

    def __enter__(self) -> 'PassContext':
        self._stack.append(self)
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        popped = self._stack.pop()
        assert popped is self

    @classmethod
    def current(cls) -> 'PassContext':
        if not cls._stack:
            cls._stack.append(PassContext())
        return cls._stack[-1]

    def set_precision(self, dtype: Optional[str] = None) -> 'PassContext':
        """'int8': add the default quantization rules; the model itself has to be float16 already, as in
        the reference, where the fused rule only fires on float16 matmuls (linear.py:115-116)."""
        if dtype == 'int8':
            from .patterns import default_patterns

            self.add_quantize_rules(default_patterns())
            self.configs['precision'] = 'float16'
        else:
            self.configs['precision'] = dtype
        return self

    def add_quantize_rules(self, patterns) -> 'PassContext':
        if patterns is None:
            self.configs['quantize_patterns'] = []
            return self
        for pat in patterns:
            if isinstance(pat, SubgraphRewriteRule):
                self.configs['quantize_patterns'].append(pat)
            elif isinstance(pat, type) and issubclass(pat, SubgraphRewriteRule):
                self.configs['quantize_patterns'].append(pat())
            else:
                raise TypeError('expect SubgraphRewriteRule instances or classes, got {!r}'.format(pat))
        return self


def module_constants(gm: fx.GraphModule, example_inputs=None) -> Dict[str, torch.Tensor]:
    """Tensors that are constant for the compiled graph: parameters / buffers reached through get_attr
    nodes, and placeholders that torch.compile bound to parameters."""
    consts: Dict[str, torch.Tensor] = {}
    placeholders = [n for n in gm.graph.nodes if n.op == 'placeholder']
    if example_inputs is not None:
        for node, value in zip(placeholders, example_inputs):
            if isinstance(value, torch.nn.Parameter):
                consts[node.name] = value.detach()
    for node in gm.graph.nodes:
        if node.op == 'get_attr':
            obj = gm
            for part in node.target.split('.'):
                obj = getattr(obj, part)
            if isinstance(obj, torch.Tensor):
                consts[node.name] = obj.detach()
    return consts


PURE_TARGETS = set()   # functions the rewrite rules insert that have no side effect (filled by the rules' module)


def drop_unused_constants(gm: fx.GraphModule) -> None:
    """Removes what a rewrite left without users: get_attr nodes and calls of the rules' own side-effect-free
    functions.  (Not fx's dead-code elimination: that also drops in-place updates whose result nobody reads, such
    as writes into a key/value cache.)"""
    for node in reversed(list(gm.graph.nodes)):
        if node.users:
            continue
        if node.op == 'get_attr' or (node.op == 'call_function' and node.target in PURE_TARGETS):
            gm.graph.erase_node(node)


def selective_quantize_pass(gm: fx.GraphModule, constants: Dict[str, torch.Tensor]) -> int:
    """Applies the context's quantize patterns (python/hidet/graph/transforms/selective_quantize.py:20-24)."""
    total = 0
    for rule in PassContext.current().configs['quantize_patterns']:
        total += rule.apply(gm, constants)
    if total:
        drop_unused_constants(gm)
        gm.graph.lint()
        gm.recompile()
    return total


def optimize(gm: fx.GraphModule, example_inputs=None) -> fx.GraphModule:
    """The slice of hidet.graph.optimize that concerns this path (python/hidet/graph/transforms/__init__.py:53-70):
    selective_quantize; variants are resolved when the quantized operators execute."""
    selective_quantize_pass(gm, module_constants(gm, example_inputs))
    return gm
