"""The reference's split-K choice, restated (python/hidet/graph/ops/quant/resolve.py:42-96)."""
import pytest

from hidet_b200.quant.resolve import resolve_k_parts
from hidet_b200.graph import PassContext, SymmetricLinearQuantizePattern, default_patterns


def test_disabled_is_one_part():
    assert resolve_k_parts([16, 4096], [4096, 4096]) == 1
    assert resolve_k_parts([2, 32, 32], [32, 32], 'disabled') == 1


def test_default_heuristic_values():
    # estimate_blocks = batch * ceil(M/64) * ceil(N/64); k_parts = min(ceil(400 / blocks), ceil(K/64))
    assert resolve_k_parts([16, 4096], [4096, 4096], 'default') == 7      # 64 blocks -> ceil(400/64) = 7
    assert resolve_k_parts([1, 4096], [4096, 11008], 'default') == 3      # 172 blocks -> 3
    assert resolve_k_parts([2048, 4096], [4096, 11008], 'default') == 1   # 5504 blocks -> 1
    assert resolve_k_parts([1, 128], [128, 64], 'default') == 2           # 1 block -> min(400, ceil(128/64)) = 2
    assert resolve_k_parts([4, 1, 64], [64, 64], 'default') == 1          # K = 64 allows one part


def test_integer_is_clamped():
    assert resolve_k_parts([1, 64], [64, 64], 0) == 1
    assert resolve_k_parts([1, 64], [64, 64], 7) == 7
    assert resolve_k_parts([1, 64], [64, 64], 100) == 32
    with pytest.raises(ValueError):
        resolve_k_parts([1, 64], [64, 64], 'fastest')


def test_pass_context_precision_switch():
    with PassContext() as ctx:
        assert ctx.configs['quantize_patterns'] == []
        ctx.set_precision('int8')
        assert ctx.configs['precision'] == 'float16'     # as in the reference (base.py:136-141)
        assert len(ctx.configs['quantize_patterns']) == len(default_patterns()) == 6  # embedding, constant right, constant left, two-step fusion, epilogue fusion, concatenation
        ctx.add_quantize_rules([SymmetricLinearQuantizePattern])
        assert len(ctx.configs['quantize_patterns']) == 7
        assert PassContext.current() is ctx
    with pytest.raises(ValueError):
        SymmetricLinearQuantizePattern(quant_type='int16')
    with pytest.raises(ValueError):
        SymmetricLinearQuantizePattern(dims=-1)


def test_the_pass_keeps_in_place_updates_nobody_reads():
    """A decoder writes keys and values into its cache in place and reads the cache, not the write's result; the
    clean-up after a rewrite must not take such writes for dead code."""
    import torch
    import torch.fx as fx

    from hidet_b200.graph.transforms import SubgraphRewriteRule, optimize

    class WritesCache(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.register_buffer('unused', torch.ones(3))

        def forward(self, cache, pos, x):
            cache.index_copy_(0, pos, x)
            return cache.sum() + self.unused.sum() * 0

    class CountsOne(SubgraphRewriteRule):
        def apply(self, gm, constants):
            return 1

    gm = fx.symbolic_trace(WritesCache())
    with PassContext() as ctx:
        ctx.add_quantize_rules([CountsOne()])
        optimize(gm)
    assert any(n.op == 'call_method' and n.target == 'index_copy_' for n in gm.graph.nodes)
    cache = torch.zeros(4, 2)
    out = gm(cache, torch.tensor([1]), torch.full((1, 2), 3.0))
    assert float(out) == 6.0 and float(cache[1, 0]) == 3.0
