"""Embedding quantization: the row-quantized table, the lookup kernel and the rewrite rule.

The reference's rule (python/hidet/graph/transforms/graph_patterns/quant/embedding.py:22-39) turns
embedding(W, ind) into take(symmetric_dequantize(wq, scale, dims=-1), ind, axis=0); the oracle restates exactly
that with its own quantize / dequantize, and the kernel must match it bit for bit.
"""
import numpy as np
import pytest
import torch
import torch.fx as fx
import torch.nn as nn
import torch.nn.functional as F

from conftest import seeded_weight

import hidet_b200
import oracle
from hidet_b200 import ffi
from hidet_b200 import graph as hg

pytestmark = pytest.mark.gpu


def oracle_lookup(table: np.ndarray, idx: np.ndarray, quant_type='int8'):
    wq, scale = oracle.symmetric_quantize(table, quant_type, -1)
    return oracle.symmetric_dequantize(wq, scale, -1)[idx], wq, scale


@pytest.mark.parametrize('vocab,dim,shape,itype', [(1000, 256, (7,), np.int64), (32000, 4096, (1, 37), np.int64), (513, 72, (3, 5), np.int32),
                                                   (64, 30, (11,), np.int32), (50, 8, (0,), np.int64)])
def test_lookup_matches_the_oracle_bit_for_bit(vocab, dim, shape, itype):
    table = seeded_weight(vocab, dim, seed=vocab + dim)
    rng = np.random.default_rng(1)
    idx = rng.integers(0, vocab, size=shape).astype(itype)
    if idx.size > 2:
        idx.flat[0], idx.flat[1] = 0, vocab - 1
    want, wq_o, scale_o = oracle_lookup(table, idx)
    wq, scale = hidet_b200.symmetric_quantize(torch.from_numpy(table).cuda(), 'int8', dims=-1)
    assert np.array_equal(wq.cpu().numpy(), wq_o) and np.array_equal(scale.cpu().numpy().view(np.int16), scale_o.view(np.int16))
    got = hidet_b200.symmetric_dequantize_take(wq, scale, torch.from_numpy(idx).cuda())
    assert tuple(got.shape) == tuple(shape) + (dim,) and got.dtype == torch.float16
    assert np.array_equal(got.cpu().numpy().view(np.int16), want.view(np.int16))
    # the same rows as the dequantize kernel gives for the whole table
    if idx.size:
        full = hidet_b200.symmetric_dequantize(wq, scale, dims=-1)
        assert torch.equal(got.reshape(-1, dim), full[torch.from_numpy(idx.reshape(-1)).long().cuda()])
    assert ffi.func('b200q_check_status')() == ffi.OK


@pytest.mark.parametrize('dtype,qtype', [(torch.bfloat16, 'int8'), (torch.float32, 'int8'), (torch.float16, 'int16')])
def test_lookup_other_types_equals_dequantize_then_take(dtype, qtype):
    table = torch.from_numpy(seeded_weight(300, 136, seed=9, dtype=np.float32)).cuda().to(dtype)
    wq, scale = hidet_b200.symmetric_quantize(table, qtype, dims=-1)
    idx = torch.randint(0, 300, (4, 9), generator=torch.Generator().manual_seed(2)).cuda()
    got = hidet_b200.symmetric_dequantize_take(wq, scale, idx)
    assert got.dtype == dtype
    assert torch.equal(got, hidet_b200.symmetric_dequantize(wq, scale, dims=-1)[idx])


def test_negative_and_out_of_range_indices():
    table = torch.from_numpy(seeded_weight(40, 64, seed=3)).cuda()
    wq, scale = hidet_b200.symmetric_quantize(table, 'int8', dims=-1)
    full = hidet_b200.symmetric_dequantize(wq, scale, dims=-1)
    idx = torch.tensor([-1, -40, 5], device='cuda')
    assert torch.equal(hidet_b200.symmetric_dequantize_take(wq, scale, idx), full[idx])
    assert ffi.func('b200q_check_status')() == ffi.OK
    out = hidet_b200.symmetric_dequantize_take(wq, scale, torch.tensor([3, 40, -41], device='cuda'))
    assert torch.equal(out[0], full[3]) and not out[1:].any()
    with pytest.raises(ffi.BackendException, match='outside its table'):
        ffi.func('b200q_check_status')()
    assert ffi.func('b200q_check_status')() == ffi.OK  # reported once, then cleared
    with pytest.raises(ValueError, match='int32 or int64'):
        hidet_b200.symmetric_dequantize_take(wq, scale, torch.tensor([1.0], device='cuda'))


class Embedder(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(500, 128)
        self.table = nn.Parameter(torch.randn(300, 128) * 0.02)
        self.fc = nn.Linear(128, 64, bias=False)

    def forward(self, ids, ids2):
        return self.fc(self.emb(ids) + F.embedding(ids2, self.table))


def test_embedding_rule_rewrites_modules_and_functional_calls():
    torch.manual_seed(4)
    model = Embedder().half().cuda().eval()
    ids = torch.randint(0, 500, (2, 9), device='cuda')
    ids2 = torch.randint(0, 300, (2, 9), device='cuda')
    want = model(ids, ids2)
    gm = fx.symbolic_trace(model)
    with hg.PassContext() as ctx:
        ctx.set_precision('int8')
        hg.optimize(gm)
    targets = [n.target for n in gm.graph.nodes if n.op == 'call_function']
    assert targets.count(hg.quantized_embedding) == 2 and targets.count(hg.quantized_matmul) == 1
    assert F.embedding not in targets and not any(n.op == 'call_module' for n in gm.graph.nodes)
    buffers = dict(gm.named_buffers())
    assert buffers['_b200q_emb_wq_0'].dtype == torch.int8 and tuple(buffers['_b200q_emb_scale_0'].shape) == (500,)
    got = gm(ids, ids2)
    assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-1)
    # only the embedding rule, as a caller of the reference would add it
    gm2 = fx.symbolic_trace(model)
    with hg.PassContext() as ctx:
        ctx.add_quantize_rules(hg.symmetric_embedding_quantize_patterns('int8'))
        hg.optimize(gm2)
    assert [n.target for n in gm2.graph.nodes if n.op == 'call_function'].count(hg.quantized_embedding) == 2
    assert any(n.op == 'call_module' for n in gm2.graph.nodes)  # the linear layer is left alone
