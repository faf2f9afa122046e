"""Operator objects, the quantization pass over fx graphs and the torch.compile backend on the GPU."""
import pytest
import torch
import torch.fx as fx
import torch.nn as nn
import torch.nn.functional as F

import hidet_b200
from hidet_b200 import graph as hg

pytestmark = pytest.mark.gpu


def test_operator_objects_follow_the_reference_contract():
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(256, 128, generator=g) * 0.02).half().cuda()
    op = hg.SymmetricQuantizationOp(w, quant_type='int8', dims=0)
    wq, scale = op.outputs
    assert op.attrs == {'dims': 0, 'quant_type': 'int8'} and op.name == 'SymmetricQuantization'
    wq2, scale2 = op.reforward([w])                      # cls(*inputs, **attrs)
    assert torch.equal(wq, wq2) and torch.equal(scale, scale2)
    wd = hg.SymmetricDeQuantizationOp(wq, scale, dims=0).outputs[0]
    assert torch.allclose(wd.float(), w.float(), atol=1e-1, rtol=1e-1)
    a = torch.randn(4, 256, generator=g).half().cuda()
    c = hg.SymmetricQuantizedMatmulOp(a, wq, scale).outputs[0]
    assert torch.equal(c, hidet_b200.symmetric_quant_matmul(a, wq, scale))
    parts = hg.SymmetricQuantizedMatmulF16I8Op(a, wq, scale, parallel_k_parts=3).outputs[0]
    assert tuple(parts.shape) == (3, 4, 128)
    with pytest.raises(ValueError):
        hg.SymmetricQuantizedMatmulF16I8Op(a, wq, scale, parallel_k_parts=2.0)


def test_later_resolve_rule_wins():
    calls = []

    @hg.register_resolve_rule(hg.SymmetricQuantizedMatmulOp)
    class Probe(hg.ResolveRule):
        def resolve(self, op):
            calls.append(op)
            return None  # fall through to the rule registered before

    try:
        a = torch.zeros(2, 64, dtype=torch.float16, device='cuda')
        wq = torch.zeros(64, 32, dtype=torch.int8, device='cuda')
        scale = torch.ones(32, dtype=torch.float16, device='cuda')
        out = hg.SymmetricQuantizedMatmulOp(a, wq, scale).outputs[0]
        assert len(calls) == 1 and tuple(out.shape) == (2, 32)
    finally:
        from hidet_b200.graph import transforms

        transforms._resolve_rules[hg.SymmetricQuantizedMatmulOp].pop()


class TwoLinears(nn.Module):
    def __init__(self):
        super().__init__()
        g = torch.Generator().manual_seed(1)
        self.w_kn = nn.Parameter((torch.randn(256, 512, generator=g) * 0.02).half())   # Hidet layout [K, N]
        self.fc = nn.Linear(512, 128, bias=True)                                      # torch layout [N, K]
        with torch.no_grad():
            self.fc.weight.copy_(torch.randn(128, 512, generator=g) * 0.02)
            self.fc.bias.copy_(torch.randn(128, generator=g) * 0.1)

    def forward(self, x):
        return self.fc(F.silu(torch.matmul(x, self.w_kn)))


def test_quantization_pass_rewrites_matmul_and_linear():
    model = TwoLinears().half().cuda().eval()
    x = torch.randn(8, 256, generator=torch.Generator().manual_seed(2)).half().cuda()
    want = model(x)
    gm = fx.symbolic_trace(model)
    with hg.PassContext() as ctx:
        ctx.set_precision('int8')
        hg.optimize(gm)
    targets = [n.target for n in gm.graph.nodes if n.op == 'call_function']
    assert targets.count(hg.quantized_matmul) == 2
    assert torch.matmul not in targets and F.linear not in targets
    assert not any(n.op == 'call_module' for n in gm.graph.nodes)
    buffers = dict(gm.named_buffers())
    assert buffers['_b200q_wq_0'].dtype == torch.int8 and tuple(buffers['_b200q_wq_0'].shape) == (256, 512)
    assert tuple(buffers['_b200q_wq_1'].shape) == (512, 128)        # the [N, K] weight, transposed once
    # per-output-channel scales of the nn.Linear weight: one per row of W[N, K]
    wq_ref, scale_ref = hidet_b200.symmetric_quantize(model.fc.weight.detach().t().contiguous(), 'int8', dims=0)
    assert torch.equal(buffers['_b200q_wq_1'], wq_ref) and torch.equal(buffers['_b200q_scale_1'], scale_ref)
    got = gm(x)
    # the reference's own acceptance for its quantized matmul against the fp16 one: atol = rtol = 2e-1
    assert torch.allclose(got.float(), want.float(), atol=2e-1, rtol=2e-1)
    # and exactly what the ops give when called by hand
    h = F.silu(hidet_b200.symmetric_quant_matmul(x, buffers['_b200q_wq_0'], buffers['_b200q_scale_0']))
    manual = hidet_b200.symmetric_quant_matmul(h, buffers['_b200q_wq_1'], buffers['_b200q_scale_1'], bias=model.fc.bias.detach())
    assert torch.equal(got, manual)   # the bias is added inside the kernel


class LeftConstant(nn.Module):
    def __init__(self):
        super().__init__()
        g = torch.Generator().manual_seed(7)
        self.w = nn.Parameter((torch.randn(96, 256, generator=g) * 0.02).half())   # W[M, K] on the left

    def forward(self, x):
        return torch.matmul(self.w, x)


def test_constant_on_the_left_is_stored_in_int8_behind_a_dequantize():
    """The reference's rule for matmul(W, x) (graph_patterns/quant/linear.py:52-84) keeps a plain matmul behind a
    dequantize, and its fused rule does not match that side."""
    model = LeftConstant().cuda().eval()
    x = torch.randn(256, 40, generator=torch.Generator().manual_seed(8)).half().cuda()
    want = model(x)
    gm = fx.symbolic_trace(model)
    with hg.PassContext() as ctx:
        ctx.set_precision('int8')
        hg.optimize(gm)
    targets = [n.target for n in gm.graph.nodes if n.op == 'call_function']
    assert targets.count(hg.dequantized_weight) == 1 and targets.count(torch.matmul) == 1 and hg.quantized_matmul not in targets
    buffers = dict(gm.named_buffers())
    assert buffers['_b200q_lwq_0'].dtype == torch.int8 and tuple(buffers['_b200q_lscale_0'].shape) == (256,)   # dims=0: one scale per column of W
    got = gm(x)
    wq, scale = hidet_b200.symmetric_quantize(model.w.detach(), 'int8', dims=0)
    assert torch.equal(got, torch.matmul(hidet_b200.symmetric_dequantize(wq, scale, dims=0), x))
    assert torch.allclose(got.float(), want.float(), atol=2e-1, rtol=2e-1)


def test_two_step_graph_is_fused():
    """matmul(x, dequant(wq, scale)) => symmetric_quant_matmul(x, wq, scale) (graph_patterns/quant/linear.py:87-124)."""
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(256, 128, generator=g) * 0.02).half().cuda()
    wq, scale = hidet_b200.symmetric_quantize(w, 'int8', dims=0)

    holder = nn.Module()
    holder.register_buffer('wq', wq)
    holder.register_buffer('scale', scale)
    graph = fx.Graph()
    x_node = graph.placeholder('x')
    wd = graph.call_function(hg.dequantized_weight, (graph.get_attr('wq'), graph.get_attr('scale')), {'dims': 0})
    graph.output(graph.call_function(torch.matmul, (x_node, wd)))
    gm = fx.GraphModule(holder, graph)
    x = torch.randn(5, 256, generator=g).half().cuda()
    unfused = gm(x)
    with hg.PassContext() as ctx:
        ctx.add_quantize_rules([hg.SymmetricQuantizeMatmulFused()])
        hg.optimize(gm)
    targets = [n.target for n in gm.graph.nodes if n.op == 'call_function']
    assert targets == [hg.quantized_matmul]
    fused = gm(x)
    assert torch.equal(fused, hidet_b200.symmetric_quant_matmul(x, wq, scale))
    assert torch.allclose(fused.float(), unfused.float(), atol=1e-2, rtol=1e-2)


def test_linear_weights_can_stay_in_torch_layout():
    model = TwoLinears().half().cuda().eval()
    x = torch.randn(8, 256, generator=torch.Generator().manual_seed(2)).half().cuda()
    gm = fx.symbolic_trace(model)
    with hg.PassContext() as ctx:
        ctx.add_quantize_rules([hg.SymmetricLinearQuantizePattern(linear_weight_layout='NK')])
        hg.optimize(gm)
    targets = [n.target for n in gm.graph.nodes if n.op == 'call_function']
    assert targets.count(hg.quantized_matmul) == 1 and targets.count(hg.quantized_linear_nk) == 1
    buffers = dict(gm.named_buffers())
    assert tuple(buffers['_b200q_wq_1'].shape) == (128, 512)   # [N, K], as torch keeps it
    # the same codes and scales as the transposed [K, N] weight quantized per column
    wq_kn, scale_kn = hidet_b200.symmetric_quantize(model.fc.weight.detach().t().contiguous(), 'int8', dims=0)
    assert torch.equal(buffers['_b200q_wq_1'], wq_kn.t()) and torch.equal(buffers['_b200q_scale_1'], scale_kn)
    got = gm(x)
    gm_kn = fx.symbolic_trace(model)
    with hg.PassContext() as ctx:
        ctx.add_quantize_rules([hg.SymmetricLinearQuantizePattern()])
        hg.optimize(gm_kn)
    assert (got.float() - gm_kn(x).float()).abs().max() < 2e-3


def test_pass_without_int8_leaves_the_graph_alone():
    model = TwoLinears().half().cuda().eval()
    gm = fx.symbolic_trace(model)
    with hg.PassContext():
        hg.optimize(gm)
    assert not any(n.target is hg.quantized_matmul for n in gm.graph.nodes)


class Block(nn.Module):
    """One Llama-style decoder block: RMSNorm, attention with separate projections, SwiGLU."""

    def __init__(self, hidden=256, heads=4, ffn=688):
        super().__init__()
        self.heads = heads
        self.q = nn.Linear(hidden, hidden, bias=False)
        self.k = nn.Linear(hidden, hidden, bias=False)
        self.v = nn.Linear(hidden, hidden, bias=False)
        self.o = nn.Linear(hidden, hidden, bias=False)
        self.gate = nn.Linear(hidden, ffn, bias=False)
        self.up = nn.Linear(hidden, ffn, bias=False)
        self.down = nn.Linear(ffn, hidden, bias=False)
        self.n1 = nn.Parameter(torch.ones(hidden))
        self.n2 = nn.Parameter(torch.ones(hidden))
        for p in self.parameters():
            if p.dim() == 2:
                nn.init.normal_(p, std=0.02)

    @staticmethod
    def rms(x, w):
        return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)).to(x.dtype) * w

    def forward(self, x):
        b, t, h = x.shape
        y = self.rms(x, self.n1)
        q, k, v = (f(y).view(b, t, self.heads, h // self.heads).transpose(1, 2) for f in (self.q, self.k, self.v))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(b, t, h)
        x = x + self.o(a)
        y = self.rms(x, self.n2)
        return x + self.down(F.silu(self.gate(y)) * self.up(y))


def test_epilogue_fusion_folds_swiglu_and_residuals_into_the_kernels():
    torch.manual_seed(5)
    model = Block().half().cuda().eval()
    x = torch.randn(2, 16, 256, device='cuda').half()
    with torch.no_grad():
        want = model(x)
    gm = fx.symbolic_trace(model)
    with hg.PassContext() as ctx:
        ctx.set_precision('int8')
        hg.optimize(gm)
    calls = [n for n in gm.graph.nodes if n.op == 'call_function' and n.target is hg.quantized_matmul]
    kinds = sorted((tuple(sorted(n.kwargs)) for n in calls))
    # q, k, v as one plain launch; o and down with the residual; gate and up as one launch with the SwiGLU pairing
    assert kinds == [(), ('activation',), ('residual',), ('residual',)]
    buffers = dict(gm.named_buffers())
    assert tuple(buffers['_b200q_gu_wq_0'].shape) == (256, 2 * 688)
    assert tuple(buffers['_b200q_cat_wq_0'].shape) == (256, 3 * 256)
    assert sum(1 for name in buffers if name.startswith('_b200q_wq_')) == 2   # o and down; the separate q, k, v, gate and up weights are gone
    with torch.no_grad():
        got = gm(x)
    assert (got.float() - want.float()).abs().max() < 5e-2
    # unfused rewrite of the same model: same result up to the float16 roundings the fusion removes
    gm2 = fx.symbolic_trace(model)
    with hg.PassContext() as ctx:
        ctx.add_quantize_rules(hg.symmetric_linear_patterns('int8', 0))
        hg.optimize(gm2)
    with torch.no_grad():
        unfused = gm2(x)
    assert sum(1 for n in gm2.graph.nodes if n.op == 'call_function' and n.target is hg.quantized_matmul) == 7
    assert (got.float() - unfused.float()).abs().max() < 2e-2


def test_torch_compile_backend_quantizes_a_decoder_block():
    hg.register()
    torch.manual_seed(3)
    model = Block().half().cuda().eval()
    x = torch.randn(1, 24, 256, device='cuda').half()
    with torch.no_grad():
        want = model(x)
        compiled = torch.compile(model, backend='hidet_b200', options={'precision': 'int8'})
        got = compiled(x)
        again = compiled(x)
    assert torch.equal(got, again)
    # the reference's acceptance for its int8 model test: atol = rtol = 0.5 (tests/models/test_quant_gpt2.py:103)
    assert torch.allclose(got.float(), want.float(), atol=0.5, rtol=0.5)
    assert (got.float() - want.float()).abs().max() < 5e-2
    # the weights really went through the quantized kernels: int8 codes differ from fp16 weights' output
    assert not torch.equal(got, want)
    # the reference's own backend name works too, and like the reference's it quantizes only when asked
    with torch.no_grad():
        as_hidet = torch.compile(model, backend='hidet', options={'precision': 'int8'})(x)
        plain = torch.compile(model, backend='hidet')(x)
    assert torch.equal(as_hidet, got)
    assert (plain.float() - want.float()).abs().max() < 2e-3


def test_compiled_graph_is_not_reused_with_another_module_s_weights():
    """torch.compile reuses a compiled graph for any module whose parameters have the same shapes and passes the
    parameters in as inputs; the quantized copies frozen at rewrite time must follow the module that is called,
    and weights written in place after compilation must be quantized again."""
    hg.register()

    def reference(lin, x):
        wq, scale = hidet_b200.symmetric_quantize(lin.weight.detach().t().contiguous(), 'int8', dims=0)
        return hidet_b200.symmetric_quant_matmul(x, wq, scale)

    torch.manual_seed(11)
    first = nn.Linear(256, 384, bias=False).half().cuda().eval()
    second = nn.Linear(256, 384, bias=False).half().cuda().eval()
    x = torch.randn(5, 256, device='cuda').half()
    with torch.no_grad():
        got_first = torch.compile(first, backend='hidet_b200', options={'precision': 'int8'})(x)
        compiled_second = torch.compile(second, backend='hidet_b200', options={'precision': 'int8'})
        got_second = compiled_second(x)
        assert torch.equal(got_first, reference(first, x))
        assert torch.equal(got_second, reference(second, x))
        assert not torch.equal(got_first, got_second)
        second.weight.mul_(0.5)
        second.weight[3, :] = 1.0
        assert torch.equal(compiled_second(x), reference(second, x))


def test_linears_of_one_input_are_merged_into_one_launch():
    """Query, key and value projections share their input: after the pass there is one quantized linear with the three
    weights side by side, and slices of its result stand where the three results stood."""
    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.q = nn.Linear(256, 256, bias=False)
            self.k = nn.Linear(256, 128, bias=False)
            self.v = nn.Linear(256, 128, bias=False)
            self.o = nn.Linear(256, 256, bias=False)

        def forward(self, x):
            q, k, v = self.q(x), self.k(x), self.v(x)
            return x + self.o(q * torch.cat((k, v), dim=-1))

    torch.manual_seed(5)
    model = Attn().half().cuda().eval()
    x = torch.randn(2, 7, 256, device='cuda').half()
    gm = fx.symbolic_trace(model)
    with torch.no_grad(), hg.PassContext() as ctx:
        ctx.set_precision('int8')
        hg.optimize(gm)
        got = gm(x)

        def qlin(lin, inp, **kw):
            wq, scale = hidet_b200.symmetric_quantize(lin.weight.detach().t().contiguous(), 'int8', dims=0)
            return hidet_b200.symmetric_quant_matmul(inp, wq, scale, **kw)

        q, k, v = qlin(model.q, x), qlin(model.k, x), qlin(model.v, x)
        want = qlin(model.o, q * torch.cat((k, v), dim=-1), residual=x)
    calls = [n for n in gm.graph.nodes if n.op == 'call_function' and n.target is hg.quantized_matmul]
    assert len(calls) == 2                                   # q | k | v in one, o (with the residual folded in)
    merged = calls[0]
    assert dict(gm.named_buffers())[merged.args[1].target].shape == (256, 512)
    # the merged launch may cut K elsewhere than the three separate ones: the last bit of a partial sum can differ
    assert (got.float() - want.float()).abs().max() <= 2e-3 * want.float().abs().max()
    assert torch.equal(got, gm(x))
