"""Parity at the full sizes of the benchmark configurations that the CPU oracle cannot reach in seconds,
and on the paths the small cases do not take: both prefill shapes, the 70B-shaped layer and every one of
its 2-, 4- and 8-way column shards, the [N, K] weight layout, the explicit split-K form at a large M, and a
quantize -> linear sequence inside one captured graph.

Where the oracle is too slow the yardstick is a plain fp32 matmul of the same dequantized operands
(tolerance 1e-3 of max |ref|: one rounding to half plus fp32 accumulation noise); the quantize kernels that
produce the operands are pinned bit for bit elsewhere (tests/test_quantize_gpu.py,
tests/test_reference_kernels_gpu.py).
"""
import numpy as np
import pytest
import torch

from conftest import seeded_activation, seeded_weight

import hidet_b200
import oracle
from hidet_b200 import ffi

pytestmark = pytest.mark.gpu

SPEC_TOL = 1e-2
TIGHT_TOL = 1e-3


def device_weight(k, n, seed):
    gen = torch.Generator(device='cuda').manual_seed(seed)
    w = (torch.randn(k, n, generator=gen, device='cuda', dtype=torch.float32) * 0.02).half()
    return hidet_b200.symmetric_quantize(w, 'int8', dims=0)


def device_activation(m, k, seed):
    gen = torch.Generator(device='cuda').manual_seed(seed)
    return torch.randn(m, k, generator=gen, device='cuda', dtype=torch.float32).half()


def fp32_reference(a, wq, scale):
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        return a.float() @ (wq.float() * scale.float())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def assert_close(c, ref, tol=TIGHT_TOL):
    err = (c.float() - ref).abs().max().item()
    top = ref.abs().max().item()
    assert err <= tol * top, 'max|err| {} vs max|ref| {}'.format(err, top)


@pytest.mark.parametrize('m,k,n', [(2048, 11008, 4096), (2048, 4096, 11008), (4, 4096, 11008), (4, 4096, 4096)])
def test_benchmark_shapes_against_fp32_matmul(m, k, n):
    wq, scale = device_weight(k, n, seed=k + n)
    a = device_activation(m, k, seed=m)
    assert_close(hidet_b200.symmetric_quant_matmul(a, wq, scale), fp32_reference(a, wq, scale))
    assert ffi.func('b200q_check_status')() == ffi.OK


@pytest.fixture(scope='module')
def layer_70b():
    """K = 8192, N = 28672 int8 weight of the 70B-shaped layer (235 MB), quantized once."""
    return device_weight(8192, 28672, seed=70)


@pytest.mark.parametrize('m', [1, 16, 256, 2048])
@pytest.mark.parametrize('ways', [1, 2, 4, 8])
def test_70b_layer_and_its_column_shards(layer_70b, m, ways):
    """Every shard of the column-parallel layer, run on this GPU exactly as rank r of `ways` runs it: its own
    contiguous [K, N / ways] weight and scale slice, written into its column range of the [M, N] output."""
    import ctypes

    from hidet_b200.runtime import workspaces

    wq, scale = layer_70b
    k, n = wq.shape
    a = device_activation(m, k, seed=m + ways)
    ref = fp32_reference(a, wq, scale)
    n_local = n // ways
    out = torch.full((m, n), float('nan'), dtype=torch.float16, device='cuda')
    for r in range(ways):
        wq_r = wq[:, r * n_local:(r + 1) * n_local].contiguous()
        scale_r = scale[r * n_local:(r + 1) * n_local].contiguous()
        table = (ctypes.c_void_p * 1)(out.data_ptr())
        ws_bytes = ffi.func('b200q_qlinear_workspace_bytes')(m, n_local, k, 0)
        ws_ptr, ws_size = workspaces.get(a.device, ws_bytes)
        ffi.func('b200q_qlinear_f16_i8_to_peers')(a.data_ptr(), wq_r.data_ptr(), scale_r.data_ptr(), table, 1, n, r * n_local, m, n_local, k,
                                                 ws_ptr, ws_size, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert_close(out, ref)
    assert ffi.func('b200q_check_status')() == ffi.OK


def test_70b_down_projection_shape():
    # the other 70B shape of the configuration: K = 28672, N = 8192
    wq, scale = device_weight(28672, 8192, seed=71)
    for m in (1, 16, 256):
        a = device_activation(m, 28672, seed=m)
        assert_close(hidet_b200.symmetric_quant_matmul(a, wq, scale), fp32_reference(a, wq, scale))
    assert ffi.func('b200q_check_status')() == ffi.OK


@pytest.mark.parametrize('m,k,n', [(4, 512, 256), (16, 4096, 1024), (1, 4096, 4096), (64, 1024, 512), (300, 2048, 768), (5, 200, 48), (16, 4096, 11008),
                                   (8, 8192, 3584), (4, 16384, 256), (3, 1024, 136), (2, 64, 16)])
def test_weight_layout_nk_against_the_oracle(m, k, n):
    w = seeded_weight(k, n, seed=k + n)
    wq, scale = oracle.symmetric_quantize(w, 'int8', 0)
    wq_nk = np.ascontiguousarray(wq.T)  # [N, K], K contiguous: what torch.nn.Linear keeps
    a = seeded_activation(m, k, seed=m)
    c = hidet_b200.symmetric_quant_matmul(torch.from_numpy(a).cuda(), torch.from_numpy(wq_nk).cuda(), torch.from_numpy(scale).cuda(),
                                          weight_layout='NK')
    assert tuple(c.shape) == (m, n)
    got = c.float().cpu().numpy()
    ref = oracle.symmetric_quant_matmul(a, wq_nk, scale, 'NK').astype(np.float32)
    exact = oracle.symmetric_quant_matmul(a, wq_nk, scale, 'NK', fused=True).astype(np.float32)
    top = max(float(np.abs(ref).max()), 1e-6)
    assert np.abs(got - ref).max() <= SPEC_TOL * top
    assert np.abs(got - exact).max() <= TIGHT_TOL * top
    # and it is the same function as the [K, N] layout on the transposed weight
    c_kn = hidet_b200.symmetric_quant_matmul(torch.from_numpy(a).cuda(), torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda())
    assert (c.float() - c_kn.float()).abs().max().item() <= TIGHT_TOL * top
    assert ffi.func('b200q_check_status')() == ffi.OK


@pytest.mark.parametrize('m,k,n', [(2048, 4096, 4096), (2048, 11008, 4096), (65, 1024, 520), (513, 4096, 11008)])
def test_weight_layout_nk_large_m_against_fp32_matmul(m, k, n):
    wq, scale = device_weight(k, n, seed=k + n)
    wq_nk = wq.t().contiguous()
    a = device_activation(m, k, seed=m)
    ref = fp32_reference(a, wq, scale)
    c = hidet_b200.symmetric_quant_matmul(a, wq_nk, scale, weight_layout='NK')
    assert_close(c, ref)
    # the two layouts are the same function of the same numbers
    assert_close(c, hidet_b200.symmetric_quant_matmul(a, wq, scale).float(), tol=1e-3)
    assert ffi.func('b200q_check_status')() == ffi.OK


@pytest.mark.parametrize('parts', [1, 3])
def test_explicit_k_parts_at_a_large_m(parts):
    m, k, n = 300, 1024, 512
    w = seeded_weight(k, n, seed=21)
    wq, scale = oracle.symmetric_quantize(w, 'int8', 0)
    a = seeded_activation(m, k, seed=22)
    c = hidet_b200.symmetric_quant_matmul_f16_i8(torch.from_numpy(a).cuda(), torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda(), parts)
    assert tuple(c.shape) == (parts, m, n)
    extent = -(-(-(-k // parts)) // 8) * 8
    for p in range(parts):
        lo, hi = min(p * extent, k), min((p + 1) * extent, k)
        ref = oracle.symmetric_quant_matmul(a, wq, scale, 'KN', lo, hi, fused=True).astype(np.float32)
        assert np.abs(c[p].float().cpu().numpy() - ref).max() <= TIGHT_TOL * max(float(np.abs(ref).max()), 1e-6)
    assert ffi.func('b200q_check_status')() == ffi.OK


def test_quantize_then_linear_inside_one_captured_graph():
    """The linear requests its weight tiles before it waits for the kernel in front of it (programmatic
    dependent launch).  That is only sound because no kernel of this library lets its dependents start
    before it has finished writing: a weight quantized by the launch directly in front must be seen whole."""
    k, n, m = 4096, 4096, 4
    gen = torch.Generator(device='cuda').manual_seed(5)
    ws = [(torch.randn(k, n, generator=gen, device='cuda', dtype=torch.float32) * 0.02).half() for _ in range(3)]
    a = device_activation(m, k, seed=6)
    wq = torch.zeros(k, n, dtype=torch.int8, device='cuda')      # one weight buffer, rewritten in front of every linear
    scale = torch.zeros(n, dtype=torch.float16, device='cuda')
    outs = [torch.empty(m, n, dtype=torch.float16, device='cuda') for _ in ws]
    lib_q = ffi.func('b200q_symmetric_quantize')

    def run():
        stream = torch.cuda.current_stream().cuda_stream
        for w, c in zip(ws, outs):
            lib_q(w.data_ptr(), wq.data_ptr(), scale.data_ptr(), k, n, ffi.F16, ffi.I8, 0, stream)
            hidet_b200.symmetric_quant_matmul(a, wq, scale, out=c)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            run()
        for c in outs:
            c.zero_()
        for _ in range(5):
            graph.replay()
        side.synchronize()
    for w, c in zip(ws, outs):
        wq_w, scale_w = hidet_b200.symmetric_quantize(w, 'int8', dims=0)
        assert torch.equal(c, hidet_b200.symmetric_quant_matmul(a, wq_w, scale_w))
    assert ffi.func('b200q_check_status')() == ffi.OK


@pytest.mark.parametrize('m,k,n,layout', [(256, 8192, 3584, 'KN'), (300, 4096, 1024, 'KN'), (300, 4096, 1024, 'NK'), (65, 2048, 144, 'KN')])
def test_large_m_kernel_with_k_split_over_ctas(m, k, n, layout):
    """A narrow problem at a few hundred rows (an eight-way column shard of the 70B layer at M = 256 is the first
    shape) would leave most SMs without a tile: K is split over several CTAs per tile, raw fp32 sums meet in the
    workspace and a second kernel finishes.  Same yardsticks as everywhere, and the same bits on every run."""
    assert ffi.func('b200q_qlinear_workspace_bytes')(m, n, k, 0) > 65536 * 4 + 2 * m * n * 4 - 1   # the split plan is on
    w = seeded_weight(k, n, seed=k + n)
    wq, scale = oracle.symmetric_quantize(w, 'int8', 0)
    a = seeded_activation(m, k, seed=m)
    a_t, scale_t = torch.from_numpy(a).cuda(), torch.from_numpy(scale).cuda()
    wq_t = torch.from_numpy(wq).cuda() if layout == 'KN' else torch.from_numpy(np.ascontiguousarray(wq.T)).cuda()
    c = hidet_b200.symmetric_quant_matmul(a_t, wq_t, scale_t, weight_layout=layout)
    assert torch.equal(c, hidet_b200.symmetric_quant_matmul(a_t, wq_t, scale_t, weight_layout=layout))
    exact = a.astype(np.float64) @ (wq.astype(np.float64) * scale.astype(np.float64))
    top = np.abs(exact).max()
    got = c.float().cpu().numpy()
    assert np.abs(got - exact).max() <= 1e-3 * top
    want = oracle.symmetric_quant_matmul(a, wq, scale)
    assert np.abs(got - want.astype(np.float64)).max() <= 1e-2 * top
    assert ffi.func('b200q_check_status')() == ffi.OK
