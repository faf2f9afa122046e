"""symmetric_quantize / symmetric_dequantize on the GPU against the CPU oracle: bit-exact."""
import numpy as np
import pytest
import torch

from conftest import seeded_weight

import hidet_b200
import oracle

pytestmark = pytest.mark.gpu


def _gpu_quantize(w_np, quant_type, dims):
    w = torch.from_numpy(w_np).cuda()
    wq, scale = hidet_b200.symmetric_quantize(w, quant_type, dims=dims)
    torch.cuda.synchronize()
    return wq.cpu().numpy(), scale.cpu().numpy()


def _assert_same(w_np, quant_type, dims, what):
    wq, scale = _gpu_quantize(w_np, quant_type, dims)
    wq_o, scale_o = oracle.symmetric_quantize(w_np, quant_type, dims)
    assert wq.dtype == wq_o.dtype and wq.shape == wq_o.shape and scale.shape == scale_o.shape, what
    bits = np.uint16 if w_np.dtype == np.float16 else np.uint32
    assert np.array_equal(scale.view(bits), scale_o.view(bits)), '{}: {} scale words differ'.format(
        what, int((scale.view(bits) != scale_o.view(bits)).sum()))
    assert np.array_equal(wq, wq_o), '{}: {} of {} codes differ'.format(what, int((wq != wq_o).sum()), wq.size)
    return wq, scale


# shapes and dims of the reference's tests (tests/operators_core/test_quantization.py:21-36,
# tests/operators_core/test_symmetric_quant.py:19-26) plus ragged and projection-like ones
@pytest.mark.parametrize('shape', [(32, 32), (64, 64), (256, 192), (67, 45), (1, 8), (8, 1), (3, 1000), (1000, 24), (513, 136)])
@pytest.mark.parametrize('dims', [0, -1])
@pytest.mark.parametrize('quant_type', ['int8', 'int16'])
def test_quantize_f16_bit_exact(shape, dims, quant_type):
    rng = np.random.default_rng(hash((shape, dims)) % 2**31)
    w = rng.standard_normal(shape).astype(np.float16)
    _assert_same(w, quant_type, dims, 'randn {} dims={} {}'.format(shape, dims, quant_type))


@pytest.mark.parametrize('k,n', [(4096, 4096), (4096, 11008), (11008, 4096)])
def test_quantize_projection_shapes_bit_exact(k, n):
    w = seeded_weight(k, n, seed=k + n)
    wq, scale = _assert_same(w, 'int8', 0, 'weight [{}, {}]'.format(k, n))
    assert int(np.abs(wq.astype(np.int32)).max()) == 127


def test_quantize_row_wise_long_rows():
    w = seeded_weight(300, 11008, seed=9)
    _assert_same(w, 'int8', -1, 'row-wise [300, 11008]')


def test_quantize_edge_values():
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((128, 64)) * 0.02).astype(np.float16)
    w[:, 0] = 0.0                       # scale 0 -> 0/0
    w[:, 1] = np.float16(-0.0)          # all negative zero
    w[:, 2] = np.abs(w[:, 2])           # one sign only
    w[:, 3] = np.float16(6e-8)          # smallest subnormal: the scale underflows to zero, w/0 = inf
    w[:, 4] = np.float16(65504.0)       # largest finite value
    w[5, 5] = np.float16(30000.0)       # an outlier that owns the scale
    w[:, 6] = np.float16(1e-3)          # a scale in the range where the division takes its correction step
    w[:, 7] = (np.arange(128) % 7 - 3).astype(np.float16)   # many exact ties
    for dims in (0, -1):
        _assert_same(w, 'int8', dims, 'edge values dims={}'.format(dims))
        _assert_same(w, 'int16', dims, 'edge values dims={} int16'.format(dims))


def special_value_weight(rows):
    """[rows, 64] f16 whose first columns hold NaN, infinities and signed zeros in the mixes that decide the
    absmax: abs is `(0 <= w) ? w : -w` and max is __hmax, so a NaN is skipped, -0 stays -0 and loses to +0."""
    rng = np.random.default_rng(14)
    w = (rng.standard_normal((rows, 64)) * 0.02).astype(np.float16)
    nan, inf = np.float16(np.nan), np.float16(np.inf)
    w[:, 0] = nan                                   # nothing but NaN: the absmax stays at the lowest finite value
    w[:, 1] = np.float16(-0.0); w[7, 1] = nan       # -0 and a NaN: absmax -0
    w[:, 2] = np.float16(-0.0); w[rows - 1, 2] = np.float16(0.0)   # one +0 among -0: absmax +0
    w[5, 3] = nan; w[rows // 2, 3] = -nan           # NaN of both signs inside ordinary values
    w[3, 4] = inf                                   # +inf owns the scale
    w[rows - 2, 5] = -inf                           # -inf does
    w[:, 6] = -np.abs(w[:, 6]) - np.float16(1e-3)   # negative values only
    w[:, 7] = np.float16(-65504.0)                  # the lowest finite value itself
    w[:, 8] = np.float16(-0.0)                      # -0 only
    w[:, 9] = np.float16(-0.0); w[1, 9] = np.float16(-6e-8)   # -0 and the negative subnormal next to it
    return w


@pytest.mark.parametrize('rows', [128, 1100])
def test_quantize_nan_inf_and_signed_zero_columns(rows):
    w = special_value_weight(rows)
    # an odd column count takes the element-wise kernels, a multiple of eight the packed ones: the same columns
    # must come out the same
    wq_v, scale_v = _gpu_quantize(w, 'int8', 0)
    wq_e, scale_e = _gpu_quantize(np.ascontiguousarray(w[:, :63]), 'int8', 0)
    assert np.array_equal(scale_v[:63].view(np.uint16), scale_e.view(np.uint16)) and np.array_equal(wq_v[:, :63], wq_e)
    for dims in (0, -1):
        _assert_same(w, 'int8', dims, 'special values rows={} dims={}'.format(rows, dims))
        _assert_same(w, 'int16', dims, 'special values rows={} dims={} int16'.format(rows, dims))
    wt = np.ascontiguousarray(w.T)          # the same columns as rows of the row-wise form
    _assert_same(wt, 'int8', -1, 'special values transposed rows={}'.format(rows))


def test_quantize_tie_heavy_grid():
    # values on a coarse grid make w / scale land exactly on .5 in many places
    rng = np.random.default_rng(12)
    w = (rng.integers(-254, 255, size=(512, 256)) / 2.0).astype(np.float16)
    w[0, :] = 127.0
    wq, _ = _assert_same(w, 'int8', 0, 'tie grid')
    # ties to even: 0.5 -> 0, 1.5 -> 2, 2.5 -> 2
    assert np.array_equal(wq[w == 0.5], np.zeros((w == 0.5).sum(), dtype=np.int8))
    assert np.array_equal(wq[w == 2.5], np.full((w == 2.5).sum(), 2, dtype=np.int8))


def test_quantize_unaligned_and_batched_views():
    rng = np.random.default_rng(13)
    base = rng.standard_normal((65, 70)).astype(np.float16)
    w = torch.from_numpy(base).cuda()[1:, 3:67]  # non-contiguous view, odd offsets
    wq, scale = hidet_b200.symmetric_quantize(w, 'int8', dims=0)
    wq_o, scale_o = oracle.symmetric_quantize(np.ascontiguousarray(base[1:, 3:67]), 'int8', 0)
    assert np.array_equal(wq.cpu().numpy(), wq_o) and np.array_equal(scale.cpu().numpy().view(np.uint16), scale_o.view(np.uint16))
    w3 = rng.standard_normal((4, 6, 40)).astype(np.float16)
    _assert_same(w3, 'int8', -1, '3-D last dim')
    _assert_same(w3, 'int8', 0, '3-D first dim')


@pytest.mark.parametrize('dims', [0, -1])
def test_quantize_f32_against_ieee_oracle(dims):
    # f32 on the GPU divides with the approximate division the reference's build flags select
    # (-prec-div=false), which is within 2 ulp of the IEEE quotient: scales agree to 2 ulp, codes differ
    # by at most one step where a quotient sits on a rounding boundary.
    rng = np.random.default_rng(14)
    w = (rng.standard_normal((300, 200)) * 0.02).astype(np.float32)
    wq, scale = _gpu_quantize(w, 'int8', dims)
    wq_o, scale_o = oracle.symmetric_quantize(w, 'int8', dims)
    d = scale.view(np.uint32).astype(np.int64) - scale_o.view(np.uint32).astype(np.int64)
    assert np.abs(d).max() <= 2
    diff = wq.astype(np.int32) - wq_o.astype(np.int32)
    assert np.abs(diff).max() <= 1 and (diff != 0).mean() < 1e-3


@pytest.mark.parametrize('dims', [0, -1])
def test_quantize_bf16_round_trip(dims):
    # tests/operators_core/test_quantization.py:21-36 runs bfloat16 too, with atol = rtol = 1e-1
    g = torch.Generator().manual_seed(15)
    w = torch.randn(64, 64, generator=g).to(torch.bfloat16).cuda()
    for qt in ('int8', 'int16'):
        wq, scale = hidet_b200.symmetric_quantize(w, qt, dims=dims)
        wd = hidet_b200.symmetric_dequantize(wq, scale, dims=dims)
        assert wd.dtype == torch.bfloat16
        assert torch.allclose(wd.float(), w.float(), atol=1e-1, rtol=1e-1)


@pytest.mark.parametrize('shape', [(32, 32), (64, 64), (67, 45), (4096, 4096), (513, 136)])
@pytest.mark.parametrize('dims', [0, -1])
def test_dequantize_bit_exact_and_round_trip(shape, dims):
    w = seeded_weight(shape[0], shape[1], seed=21, std=1.0)
    wq_o, scale_o = oracle.symmetric_quantize(w, 'int8', dims)
    wd = hidet_b200.symmetric_dequantize(torch.from_numpy(wq_o).cuda(), torch.from_numpy(scale_o).cuda(), dims=dims)
    wd_o = oracle.symmetric_dequantize(wq_o, scale_o, dims)
    assert np.array_equal(wd.cpu().numpy().view(np.uint16), wd_o.view(np.uint16))
    # the reference's own acceptance test: quantize -> dequantize within atol = rtol = 1e-1
    assert np.allclose(wd_o.astype(np.float32), w.astype(np.float32), atol=1e-1, rtol=1e-1)


def test_quantize_commutes_with_column_sharding():
    w = seeded_weight(1024, 512, seed=22)
    wq, scale = _gpu_quantize(w, 'int8', 0)
    for g in (2, 4, 8):
        step = 512 // g
        for r in range(g):
            wq_r, scale_r = _gpu_quantize(np.ascontiguousarray(w[:, r * step:(r + 1) * step]), 'int8', 0)
            assert np.array_equal(wq_r, wq[:, r * step:(r + 1) * step])
            assert np.array_equal(scale_r.view(np.uint16), scale[r * step:(r + 1) * step].view(np.uint16))


def test_quantize_rejects_bad_arguments():
    w = torch.zeros(8, 8, dtype=torch.float16, device='cuda')
    with pytest.raises(ValueError):
        hidet_b200.symmetric_quantize(w, 'int4', dims=0)
    with pytest.raises(ValueError):
        hidet_b200.symmetric_quantize(w.to(torch.int32), 'int8', dims=0)
    with pytest.raises(ValueError):
        hidet_b200.symmetric_quantize(w, 'int8', dims=2)
    wq, scale = hidet_b200.symmetric_quantize(w, 'int8', dims=0)
    with pytest.raises(ValueError):
        hidet_b200.symmetric_dequantize(wq, scale[:4], dims=0)
