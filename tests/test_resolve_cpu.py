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
        assert len(ctx.configs['quantize_patterns']) == len(default_patterns()) == 5  # embedding, constant right, constant left, two-step fusion, epilogue fusion
        ctx.add_quantize_rules([SymmetricLinearQuantizePattern])
        assert len(ctx.configs['quantize_patterns']) == 6
        assert PassContext.current() is ctx
    with pytest.raises(ValueError):
        SymmetricLinearQuantizePattern(quant_type='int16')
    with pytest.raises(ValueError):
        SymmetricLinearQuantizePattern(dims=-1)
