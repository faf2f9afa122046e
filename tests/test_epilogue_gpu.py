"""The fused epilogue of the quantized linear: bias, SwiGLU pairing, residual.

The reference reaches the same graph by fusing the element-wise operators that follow its matmul
(python/hidet/graph/transforms/fuse_operator.py); there every operator rounds to float16, here the kernel rounds
once.  The yardstick is float64 arithmetic on the dequantized operands (numpy), tolerance 1e-3 of the largest
result, and the unfused sequence of this library's own kernel plus torch element-wise operators, which must
agree to float16 rounding of each of its steps.
"""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from conftest import seeded_activation, seeded_weight

import hidet_b200
import oracle
from hidet_b200 import ffi
from hidet_b200.quant import interleave_gate_up

pytestmark = pytest.mark.gpu

# small-M kernel: cluster split, one CTA per tile, splits through the workspace; large-M kernel: short and tall tiles,
# and (the last two) K split over several CTAs per tile with the epilogue in the reduce kernel
SHAPES = [(1, 4096, 4096), (4, 1024, 512), (16, 4096, 1024), (3, 512, 19008), (4, 16384, 256), (12, 2048, 16), (40, 512, 256),
          (300, 1024, 768), (2048, 512, 1024), (300, 4096, 1024), (100, 8192, 528)]


def float64_sums(a, wq, scale):
    return a.astype(np.float64) @ (wq.astype(np.float64) * scale.astype(np.float64))


def silu64(x):
    return x / (1.0 + np.exp(-x))


def to_cuda(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(x)).cuda() for x in arrays]


@pytest.mark.parametrize('m,k,n', SHAPES)
@pytest.mark.parametrize('with_bias,with_res,act', [(True, False, None), (False, True, None), (False, False, 'silu_mul'), (True, True, 'silu_mul'),
                                                    (True, True, None)])
def test_fused_epilogue(m, k, n, with_bias, with_res, act):
    w = seeded_weight(k, n, seed=k + n)
    wq, scale = oracle.symmetric_quantize(w, 'int8', 0)
    a = seeded_activation(m, k, seed=m)
    rng = np.random.default_rng(n)
    bias = (rng.standard_normal(n) * 0.5).astype(np.float16) if with_bias else None
    n_out = n // 2 if act else n
    res = rng.standard_normal((m, n_out)).astype(np.float16) if with_res else None

    y = float64_sums(a, wq, scale)
    if bias is not None:
        y = y + bias.astype(np.float64)
    if act:
        y = silu64(y[:, 0::2]) * y[:, 1::2]
    if res is not None:
        y = y + res.astype(np.float64)

    a_t, wq_t, scale_t = to_cuda(a, wq, scale)
    bias_t = to_cuda(bias)[0] if with_bias else None
    res_t = to_cuda(res)[0] if with_res else None
    got = hidet_b200.symmetric_quant_matmul(a_t, wq_t, scale_t, bias=bias_t, residual=res_t, activation=act)
    assert tuple(got.shape) == (m, n_out) and got.dtype == torch.float16
    top = max(float(np.abs(y).max()), 1e-6)
    assert np.abs(got.float().cpu().numpy() - y).max() <= 1e-3 * top

    # the same graph, unfused: this library's plain kernel, then torch's element-wise operators in float16
    u = hidet_b200.symmetric_quant_matmul(a_t, wq_t, scale_t)
    if bias_t is not None:
        u = u + bias_t
    if act:
        u = F.silu(u[:, 0::2]) * u[:, 1::2]
    if res_t is not None:
        u = u + res_t
    assert (got.float() - u.float()).abs().max().item() <= 4e-3 * top
    assert ffi.func('b200q_check_status')() == ffi.OK


def test_gate_up_interleaving_commutes_with_quantization():
    k, f = 512, 384
    gate, up = seeded_weight(k, f, seed=1), seeded_weight(k, f, seed=2)
    g_t, u_t = to_cuda(gate, up)
    wq_g, s_g = hidet_b200.symmetric_quantize(g_t, 'int8', dims=0)
    wq_u, s_u = hidet_b200.symmetric_quantize(u_t, 'int8', dims=0)
    wq_gu, s_gu = hidet_b200.symmetric_quantize(interleave_gate_up(g_t, u_t), 'int8', dims=0)
    assert torch.equal(wq_gu, interleave_gate_up(wq_g, wq_u)) and torch.equal(s_gu, interleave_gate_up(s_g, s_u))
    a = to_cuda(seeded_activation(5, k, seed=3))[0]
    fused = hidet_b200.symmetric_quant_matmul(a, wq_gu, s_gu, activation='silu_mul')
    separate = F.silu(hidet_b200.symmetric_quant_matmul(a, wq_g, s_g)) * hidet_b200.symmetric_quant_matmul(a, wq_u, s_u)
    assert (fused.float() - separate.float()).abs().max().item() <= 4e-3 * separate.float().abs().max().item()


def test_fused_epilogue_argument_checks():
    a = torch.zeros(4, 64, dtype=torch.float16, device='cuda')
    wq = torch.zeros(64, 32, dtype=torch.int8, device='cuda')
    scale = torch.ones(32, dtype=torch.float16, device='cuda')
    with pytest.raises(ValueError, match='activation must be'):
        hidet_b200.symmetric_quant_matmul(a, wq, scale, activation='gelu')
    with pytest.raises(ValueError, match='bias of shape'):
        hidet_b200.symmetric_quant_matmul(a, wq, scale, bias=torch.zeros(16, dtype=torch.float16, device='cuda'))
    with pytest.raises(ValueError, match='residual of shape'):
        hidet_b200.symmetric_quant_matmul(a, wq, scale, residual=torch.zeros(4, 32, dtype=torch.float16, device='cuda'), activation='silu_mul')
    with pytest.raises(ValueError, match="weight_layout='KN' only"):
        hidet_b200.symmetric_quant_matmul(a, wq.t().contiguous(), scale, weight_layout='NK', bias=torch.zeros(32, dtype=torch.float16, device='cuda'))
    ep = ffi.Epilogue(None, None, 0, 7)
    import ctypes

    out = torch.empty(4, 32, dtype=torch.float16, device='cuda')
    with pytest.raises(ffi.BackendException, match='unknown activation 7'):
        ffi.func('b200q_qlinear_f16_i8_fused')(a.data_ptr(), wq.data_ptr(), scale.data_ptr(), out.data_ptr(), 4, 32, 64, 0, ctypes.byref(ep), None, 0,
                                              torch.cuda.current_stream().cuda_stream)
