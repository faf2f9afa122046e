"""torch.compile backend: ``torch.compile(model, backend='hidet_b200', options={'precision': 'int8'})``.

The reference's backend (python/hidet/graph/frontend/torch/dynamo_backends.py:144-175) opens a fresh
PassContext and offers no way to switch quantization on; this backend takes it as an option.  The fx
graph is rewritten by the quantization pass (float16 linear layers with constant weights become
calls into libhidet_b200q.so) and otherwise runs as captured: only the quantized-linear path is
replaced.  Weights are frozen when the graph is rewritten, as the reference freezes them into graph constants;
a call with other parameter tensors (another module of the same shapes, or weights written since) is rewritten anew.
"""
from __future__ import annotations

import copy
from typing import Any, Dict, List, Optional

import torch
import torch.fx as fx

from .transforms import PassContext, optimize

_registered = False


_MAX_VARIANTS = 8


def _rewrite(gm: fx.GraphModule, inputs, precision):
    with PassContext() as ctx:
        ctx.set_precision(precision)
        optimize(gm, inputs)
    return gm.forward


def hidet_b200_backend(gm: fx.GraphModule, example_inputs: List[Any], options: Optional[Dict[str, Any]] = None, **kwargs):
    options = dict(options or {})
    options.update(kwargs.get('options') or {})
    precision = options.get('precision', 'int8')
    # torch.compile hands a module's parameters to the graph as inputs and reuses the compiled graph for any
    # module whose parameters have the same shapes.  The rewrite freezes the parameters it quantizes, so the
    # compiled callable checks on every call that it is given the very tensors it froze (same storage, not
    # written since) and rewrites a fresh copy of the captured graph when it is not.
    frozen = [i for i, v in enumerate(example_inputs) if isinstance(v, torch.nn.Parameter)]
    if not frozen:
        return _rewrite(gm, example_inputs, precision)
    pristine = copy.deepcopy(gm)

    def key(args):
        return tuple((args[i].data_ptr(), args[i]._version) for i in frozen)

    variants = {key(example_inputs): _rewrite(gm, example_inputs, precision)}

    def run(*args):
        k = key(args)
        fn = variants.get(k)
        if fn is None:
            if len(variants) >= _MAX_VARIANTS:
                variants.pop(next(iter(variants)))
            fn = variants[k] = _rewrite(copy.deepcopy(pristine), list(args), precision)
        return fn(*args)

    return run


def hidet_backend(gm: fx.GraphModule, example_inputs: List[Any], options: Optional[Dict[str, Any]] = None, **kwargs):
    """The same backend under the reference's own name.  Like the reference's, it quantizes nothing unless asked:
    torch.compile(model, backend='hidet', options={'precision': 'int8'})."""
    options = dict(options or {})
    options.update(kwargs.pop('options', None) or {})
    options.setdefault('precision', None)
    return hidet_b200_backend(gm, example_inputs, options=options)


def register() -> None:
    """Makes backend='hidet_b200' known to torch.compile and, where no package has claimed the reference's
    backend name, backend='hidet' as well, so that code written for the reference keeps working (idempotent)."""
    global _registered
    if _registered:
        return
    from torch._dynamo import list_backends, register_backend

    register_backend(name='hidet_b200', compiler_fn=hidet_b200_backend)
    if 'hidet' not in list_backends(exclude_tags=()):
        register_backend(name='hidet', compiler_fn=hidet_backend)
    _registered = True
