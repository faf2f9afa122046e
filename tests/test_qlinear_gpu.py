"""The f16 x int8 quantized matmul on the GPU against the CPU oracle.

Tolerance: max |err| <= 1e-2 * max |ref| against the reference's dequantize-then-matmul value (the bar
the benchmark specification sets), and a much tighter bound against the exact-sum value the kernels
aim at (one rounding to half: 2^-11 relative, plus fp32 accumulation noise).
"""
import numpy as np
import pytest
import torch

from conftest import seeded_activation, seeded_weight

import hidet_b200
import oracle
from hidet_b200 import ffi

pytestmark = pytest.mark.gpu

SPEC_TOL = 1e-2   # of max |ref|
TIGHT_TOL = 1e-3  # of max |ref|, against the exact-sum oracle


def _quantized(k, n, seed=0):
    w = seeded_weight(k, n, seed=seed)
    return oracle.symmetric_quantize(w, 'int8', 0)


def _check(a_np, wq_np, scale_np, c_gpu, layout='KN', k_begin=0, k_end=None):
    c = c_gpu.float().cpu().numpy().reshape(-1, c_gpu.shape[-1])
    a2 = a_np.reshape(-1, a_np.shape[-1])
    ref = oracle.symmetric_quant_matmul(a2, wq_np, scale_np, layout, k_begin, k_end).astype(np.float32)
    exact = oracle.symmetric_quant_matmul(a2, wq_np, scale_np, layout, k_begin, k_end, fused=True).astype(np.float32)
    scale_ref = max(float(np.abs(ref).max()), 1e-6)
    err = float(np.abs(c - ref).max())
    err_exact = float(np.abs(c - exact).max())
    assert err <= SPEC_TOL * scale_ref, 'max|err| {} vs max|ref| {}'.format(err, scale_ref)
    assert err_exact <= TIGHT_TOL * scale_ref, 'max|err| {} vs exact-sum oracle, max|ref| {}'.format(err_exact, scale_ref)


# decode shapes of the benchmark (M in {1, 4, 16}, K = 4096, N in {4096, 11008}) and the reference's own
# test shapes (tests/operators_core/test_quantization.py:39-47)
@pytest.mark.parametrize('m,k,n', [(1, 4096, 4096), (4, 4096, 4096), (16, 4096, 4096), (1, 4096, 11008), (16, 4096, 11008),
                                   (16, 11008, 4096), (3, 512, 256), (7, 1024, 384), (16, 64, 128), (1, 8, 16), (5, 200, 48),
                                   (8, 8192, 3584), (9, 16384, 256), (2, 28672, 1024), (12, 2048, 16), (16, 8192, 1024)])
def test_qlinear_small_m(m, k, n):
    wq, scale = _quantized(k, n, seed=m + k)
    a = seeded_activation(m, k, seed=n)
    c = hidet_b200.symmetric_quant_matmul(torch.from_numpy(a).cuda(), torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda())
    assert c.shape == (m, n) and c.dtype == torch.float16
    _check(a, wq, scale, c)


@pytest.mark.parametrize('shape_a,shape_w', [((2, 32, 32), (32, 32)), ((1, 64, 64), (64, 128))])
def test_qlinear_reference_test_shapes(shape_a, shape_w):
    rng = np.random.default_rng(3)
    a = rng.standard_normal(shape_a).astype(np.float16)
    w = rng.standard_normal(shape_w).astype(np.float16)
    wq, scale = oracle.symmetric_quantize(w, 'int8', 0)
    c = hidet_b200.symmetric_quant_matmul(torch.from_numpy(a).cuda(), torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda())
    assert tuple(c.shape) == shape_a[:-1] + (shape_w[1],)
    _check(a, wq, scale, c)
    # the reference's own acceptance: against the fp16 matmul with the unquantized weight, atol = rtol = 2e-1
    want = a.astype(np.float32) @ w.astype(np.float32)
    assert np.allclose(c.float().cpu().numpy(), want, atol=2e-1, rtol=2e-1)


@pytest.mark.parametrize('m,k,n', [(17, 512, 256), (64, 1024, 512), (200, 640, 384), (256, 4096, 1024), (33, 64, 16), (100, 72, 4096),
                                   (300, 1024, 2048), (513, 512, 19008), (1000, 264, 272)])
def test_qlinear_larger_m(m, k, n):
    wq, scale = _quantized(k, n, seed=5)
    a = seeded_activation(m, k, seed=6)
    c = hidet_b200.symmetric_quant_matmul(torch.from_numpy(a).cuda(), torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda())
    _check(a, wq, scale, c)


@pytest.mark.parametrize('m,k,n', [(3, 100, 36), (4, 64, 20), (2, 36, 16), (1, 4098, 130)])
def test_qlinear_unaligned_shapes(m, k, n):
    # rows that are not 16-byte multiples take the shape-agnostic kernel
    wq, scale = _quantized(k, n, seed=7)
    a = seeded_activation(m, k, seed=8)
    c = hidet_b200.symmetric_quant_matmul(torch.from_numpy(a).cuda(), torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda())
    _check(a, wq, scale, c)


@pytest.mark.parametrize('parts', [1, 2, 3, 5, 16])
def test_qlinear_explicit_k_parts(parts):
    m, k, n = 8, 1000, 256
    wq, scale = _quantized(k, n, seed=9)
    a = seeded_activation(m, k, seed=10)
    c = hidet_b200.symmetric_quant_matmul_f16_i8(torch.from_numpy(a).cuda(), torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda(), parts)
    assert tuple(c.shape) == (parts, m, n)
    extent = -(-(-(-k // parts)) // 8) * 8  # ceil(ceil(K / parts) / 8) * 8, python/hidet/graph/ops/quant/matmul_f16_i8.py:165
    for p in range(parts):
        lo, hi = min(p * extent, k), min((p + 1) * extent, k)
        if lo == hi:
            assert not c[p].any()
        else:
            _check(a, wq, scale, c[p], k_begin=lo, k_end=hi)
    # what the resolve rule does with it: .sum(0)
    total = c.float().sum(0).half()
    ref = oracle.symmetric_quant_matmul(a, wq, scale).astype(np.float32)
    assert np.abs(total.float().cpu().numpy() - ref).max() <= SPEC_TOL * np.abs(ref).max()


def test_qlinear_atomic_form_is_deterministic():
    m, k, n = 16, 4096, 4096
    wq, scale = _quantized(k, n, seed=11)
    a = seeded_activation(m, k, seed=12)
    args = (torch.from_numpy(a).cuda(), torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda())
    c1 = hidet_b200.symmetric_quant_matmul_atomic_f16_i8(*args, parallel_k_parts=4)
    c2 = hidet_b200.symmetric_quant_matmul_atomic_f16_i8(*args, parallel_k_parts=8)
    c3 = hidet_b200.symmetric_quant_matmul(*args)
    assert torch.equal(c1, c2) and torch.equal(c1, c3)
    _check(a, wq, scale, c1)


def test_qlinear_one_hot_rows_return_dequantized_weight_rows():
    # size-independent exactness check at a full benchmark shape: a one-hot activation row selects one
    # weight row, and a sum of one term has no accumulation error, so the output must equal the
    # dequantize kernel's row bit for bit
    k, n = 4096, 11008
    wq, scale = _quantized(k, n, seed=13)
    rows = [0, 1, 63, 64, 1000, 2047, 2048, 4095, 17, 333, 4000, 2500, 129, 511, 512, 3071]
    a = np.zeros((16, k), dtype=np.float16)
    for i, r in enumerate(rows):
        a[i, r] = 1.0
    wq_t, scale_t = torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda()
    c = hidet_b200.symmetric_quant_matmul(torch.from_numpy(a).cuda(), wq_t, scale_t)
    wd = hidet_b200.symmetric_dequantize(wq_t, scale_t, dims=0)
    assert torch.equal(c, wd[rows])


def test_qlinear_power_of_two_scaling_and_column_permutation():
    m, k, n = 4, 4096, 4096
    wq, scale = _quantized(k, n, seed=14)
    a = seeded_activation(m, k, seed=15)
    a_t, wq_t, scale_t = torch.from_numpy(a).cuda(), torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda()
    c = hidet_b200.symmetric_quant_matmul(a_t, wq_t, scale_t)
    c2 = hidet_b200.symmetric_quant_matmul(a_t * 2, wq_t, scale_t)
    # doubling is exact in every step except the last rounding of results that are subnormal in half
    normal = c.abs() >= 2.0 ** -13
    assert torch.equal(c2[normal], (c * 2)[normal])
    assert ((c2.float() - 2 * c.float()).abs() <= 2.0 ** -24).all()
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(1)).cuda()
    cp = hidet_b200.symmetric_quant_matmul(a_t, wq_t[:, perm].contiguous(), scale_t[perm].contiguous())
    assert torch.equal(cp, c[:, perm])


def test_qlinear_full_prefill_shape_against_fp32_matmul():
    # too large for the CPU oracle in seconds: compare with a plain fp32 matmul of the same dequantized operands
    m, k, n = 2048, 4096, 11008
    wq, scale = _quantized(k, n, seed=16)
    a_t = torch.from_numpy(seeded_activation(m, k, seed=17)).cuda()
    wq_t, scale_t = torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda()
    c = hidet_b200.symmetric_quant_matmul(a_t, wq_t, scale_t)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref = a_t.float() @ (wq_t.float() * scale_t.float())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    err = (c.float() - ref).abs().max().item()
    assert err <= TIGHT_TOL * ref.abs().max().item()


def test_qlinear_empty_and_degenerate():
    wq, scale = _quantized(64, 32, seed=18)
    wq_t, scale_t = torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda()
    a0 = torch.zeros(0, 64, dtype=torch.float16, device='cuda')
    assert tuple(hidet_b200.symmetric_quant_matmul(a0, wq_t, scale_t).shape) == (0, 32)


def test_qlinear_argument_checks_follow_the_reference():
    a = torch.zeros(4, 64, dtype=torch.float16, device='cuda')
    wq = torch.zeros(64, 32, dtype=torch.int8, device='cuda')
    scale = torch.ones(32, dtype=torch.float16, device='cuda')
    with pytest.raises(ValueError, match='at least 2 dimensions'):
        hidet_b200.symmetric_quant_matmul(a[0], wq, scale)
    with pytest.raises(ValueError, match='only support float16, int8'):
        hidet_b200.symmetric_quant_matmul(a.float(), wq, scale)
    with pytest.raises(ValueError, match='multiple of 2'):
        hidet_b200.symmetric_quant_matmul(a[:, :63], wq[:63], scale)
    with pytest.raises(ValueError, match='Matrix multiplication expect'):
        hidet_b200.symmetric_quant_matmul(a, wq[:32], scale)
    with pytest.raises(ValueError, match='parallel_k_parts must be an integer'):
        hidet_b200.symmetric_quant_matmul_f16_i8(a, wq, scale, 1.5)
    # a too small workspace is reported, not overrun
    with pytest.raises(ffi.BackendException, match='workspace'):
        # a narrow, deep problem is split over more CTAs than a cluster holds and needs the workspace
        m, n, k = 4, 256, 16384
        assert ffi.func('b200q_qlinear_workspace_bytes')(m, n, k, 0) > 256
        big_a = torch.zeros(m, k, dtype=torch.float16, device='cuda')
        big_w = torch.zeros(k, n, dtype=torch.int8, device='cuda')
        big_s = torch.ones(n, dtype=torch.float16, device='cuda')
        out = torch.empty(m, n, dtype=torch.float16, device='cuda')
        tiny = torch.zeros(256, dtype=torch.uint8, device='cuda')
        ffi.func('b200q_qlinear_f16_i8')(big_a.data_ptr(), big_w.data_ptr(), big_s.data_ptr(), out.data_ptr(), m, n, k, 0,
                                         tiny.data_ptr(), tiny.numel(), torch.cuda.current_stream().cuda_stream)
    assert ffi.func('b200q_check_status')() == ffi.OK


def _to_destinations(a, wq, scale, dsts, ldc, col0):
    import ctypes

    from hidet_b200.runtime import workspaces

    m, k = a.shape
    n = wq.shape[1]
    table = (ctypes.c_void_p * len(dsts))(*[d.data_ptr() for d in dsts])
    ws_bytes = ffi.func('b200q_qlinear_workspace_bytes')(m, n, k, 0)
    ws_ptr, ws_size = workspaces.get(a.device, ws_bytes)
    ffi.func('b200q_qlinear_f16_i8_to_peers')(a.data_ptr(), wq.data_ptr(), scale.data_ptr(), table, len(dsts), ldc, col0, m, n, k,
                                             ws_ptr, ws_size, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize('m,k,n', [(1, 1024, 256), (16, 8192, 1792), (32, 512, 128), (300, 2048, 256), (40, 8192, 4096), (300, 4096, 1024)])
def test_qlinear_into_a_column_range_of_wider_outputs(m, k, n):
    """The column-parallel entry point on one GPU: every destination gets the plain result in its columns and
    nothing outside them, from either kernel."""
    wq, scale = _quantized(k, n, seed=5)
    a = torch.from_numpy(seeded_activation(m, k, seed=6)).cuda()
    wq_t, scale_t = torch.from_numpy(wq).cuda(), torch.from_numpy(scale).cuda()
    want = hidet_b200.symmetric_quant_matmul(a, wq_t, scale_t)
    ldc, col0 = 2 * n + 64, n + 32
    count = 3
    dsts = [torch.full((m, ldc), -7.0, dtype=torch.float16, device='cuda') for _ in range(count)]
    _to_destinations(a, wq_t, scale_t, dsts, ldc, col0)
    torch.cuda.synchronize()
    for d in dsts:
        assert torch.equal(d[:, col0:col0 + n], want)
        assert bool((d[:, :col0] == -7.0).all()) and bool((d[:, col0 + n:] == -7.0).all())
    assert ffi.func('b200q_check_status')() == ffi.OK


def test_multicast_entry_point_refuses_what_it_does_not_serve():
    """The multicast delivery needs an NVLink multicast mapping, which one GPU does not have; what can be checked
    here is that the entry point takes large M only and says where small M goes."""
    f = ffi.func('b200q_qlinear_f16_i8_to_multicast')
    a = torch.zeros(16, 512, dtype=torch.float16, device='cuda')
    wq = torch.zeros(512, 128, dtype=torch.int8, device='cuda')
    scale = torch.ones(128, dtype=torch.float16, device='cuda')
    out = torch.zeros(16, 128, dtype=torch.float16, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    with pytest.raises(ffi.BackendException, match='to_peers') as e:
        f(a.data_ptr(), wq.data_ptr(), scale.data_ptr(), out.data_ptr(), 128, 0, 16, 128, 512, None, 0, stream)
    assert e.value.status == ffi.UNSUPPORTED
    with pytest.raises(ffi.BackendException, match='null destination'):
        f(a.data_ptr(), wq.data_ptr(), scale.data_ptr(), None, 128, 0, 16, 128, 512, None, 0, stream)
    with pytest.raises(ffi.BackendException, match='do not fit'):
        f(a.data_ptr(), wq.data_ptr(), scale.data_ptr(), out.data_ptr(), 64, 0, 16, 128, 512, None, 0, stream)


def test_push_columns_copies_one_column_range_and_nothing_else():
    import ctypes

    rows, ld, col0, cols = 37, 512, 96, 200
    src = torch.randn(rows, ld, device='cuda').half()
    dsts = [torch.full((rows, ld), -3.0, dtype=torch.float16, device='cuda') for _ in range(2)]
    table = (ctypes.c_void_p * 3)(src.data_ptr(), dsts[0].data_ptr(), dsts[1].data_ptr())  # the first entry is the source itself
    before = src.clone()
    ffi.func('b200q_push_columns')(src.data_ptr(), table, 3, rows, cols, ld, col0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(src, before)
    for d in dsts:
        assert torch.equal(d[:, col0:col0 + cols], src[:, col0:col0 + cols])
        assert bool((d[:, :col0] == -3.0).all()) and bool((d[:, col0 + cols:] == -3.0).all())
    with pytest.raises(ffi.BackendException, match='do not fit'):
        ffi.func('b200q_push_columns')(src.data_ptr(), table, 3, rows, cols, ld, ld - cols + 1, torch.cuda.current_stream().cuda_stream)
