"""4-bit weights with group scales and zero points (w4a16) on the GPU against the oracle, through the host layer that
mirrors the reference's test programs (tests/cute_kernel/test_quant_linear.py)."""
import numpy as np
import pytest
import torch

import hidet_b200
from hidet_b200 import ffi
from hidet_b200.quant import cast_f16_to_u4, cast_u4_to_f16, preprocess_weight, w4a16_linear
from oracle import subbyte

pytestmark = pytest.mark.gpu


def test_pack_and_unpack_match_the_oracle_bit_for_bit():
    g = torch.Generator().manual_seed(0)
    w = torch.randint(0, 16, (130, 264), generator=g).to(torch.float16)
    w[0, :4] = torch.tensor([17.9, -1.0, 15.0, 0.0])
    packed = cast_f16_to_u4(w.cuda())
    assert packed.dtype == torch.int32 and tuple(packed.shape) == (130, 33)
    want = subbyte.pack_u4(w.numpy())
    assert np.array_equal(packed.cpu().numpy().view(np.uint8), want)
    back = cast_u4_to_f16(packed)
    assert np.array_equal(back.cpu().numpy().astype(np.uint8), subbyte.unpack_u4(want))
    assert preprocess_weight(packed) is packed


@pytest.mark.parametrize('problem_size', [[1, 4096, 4096], [1, 4096, 12288], [1, 12288, 4096]])
@pytest.mark.parametrize('with_zp', [True, False])
def test_quant_linear_on_the_reference_s_test_data(problem_size, with_zp):
    """The reference's own test (tests/cute_kernel/test_quant_linear.py:53-85), same shapes, group size and data
    distribution; on such data every sum is exact, so the result must equal torch's to the bit."""
    gsize = 128
    m, n, k = problem_size
    gen = torch.Generator(device='cuda').manual_seed(m + n + k)
    a = torch.randint(-3, 3, (m, k), device='cuda', generator=gen).to(torch.float16)
    b = torch.randint(0, 3, (k, n), device='cuda', generator=gen).to(torch.float16)
    scale = torch.randint(0, 2, (k // gsize, n), device='cuda', generator=gen).to(torch.float16)
    zeros = torch.randint(0, 3, (k // gsize, n), device='cuda', generator=gen).to(torch.float16)
    bq = cast_f16_to_u4(b)
    assert torch.equal(cast_u4_to_f16(bq), b)
    linear = w4a16_linear('w4a16', k, n, gsize, with_zp=with_zp)
    c = linear(a, preprocess_weight(bq), scale, zeros)
    b2 = b.float().view(k // gsize, gsize, n)
    b3 = scale.float().view(k // gsize, 1, n) * ((b2 - zeros.float().view(k // gsize, 1, n)) if with_zp else b2)
    c2 = a.float() @ b3.view(k, n)
    np.testing.assert_allclose(actual=c.float().cpu().numpy(), desired=c2.cpu().numpy(), rtol=2e-3)
    assert torch.equal(c, c2.half())
    assert torch.equal(c, linear(a, bq, scale, zeros))   # the same on every run


@pytest.mark.parametrize('m,n,k,gsize', [(1, 4096, 4096, 128), (3, 264, 1024, 64), (8, 11008, 4096, 128), (33, 512, 768, 256), (5, 8, 64, 64)])
@pytest.mark.parametrize('with_zp', [True, False])
def test_quant_linear_on_real_valued_scales(m, n, k, gsize, with_zp):
    rng = np.random.default_rng(m * 7 + n)
    a = rng.standard_normal((m, k)).astype(np.float16)
    codes = rng.integers(0, 16, (k, n)).astype(np.float16)
    scale = (rng.random((k // gsize, n)) * 0.01 + 0.002).astype(np.float16)
    zeros = (rng.random((k // gsize, n)) * 15).astype(np.float16)
    bq = cast_f16_to_u4(torch.from_numpy(codes).cuda())
    linear = w4a16_linear('w4a16', k, n, gsize, with_zp=with_zp)
    c = linear(torch.from_numpy(a).cuda(), bq, torch.from_numpy(scale).cuda(), torch.from_numpy(zeros).cuda()).float().cpu().numpy()
    packed = subbyte.pack_u4(codes)
    exact = subbyte.w4a16_linear(a, packed, scale, zeros if with_zp else None, gsize)
    as_reference = subbyte.w4a16_linear(a, packed, scale, zeros if with_zp else None, gsize, f16_steps=True)
    top = np.abs(exact).max()
    assert np.abs(c - exact).max() <= 1e-3 * top          # fp32 sums, one rounding to f16
    assert np.abs(c - as_reference).max() <= 1e-2 * top   # the reference rounds every weight to f16 first
    assert np.isfinite(c).all()


def test_quant_linear_argument_errors():
    f = ffi.func('b200q_qlinear_f16_u4')
    with pytest.raises(ffi.BackendException, match='multiple of the group size'):
        f(1, 1, 1, None, 1, 1, 64, 100, 64, None, 0, None)
    with pytest.raises(ffi.BackendException, match='multiple of 8'):
        f(1, 1, 1, None, 1, 1, 12, 64, 64, None, 0, None)
    a = torch.zeros(2, 64, dtype=torch.float16, device='cuda')
    q = torch.zeros(64, 2, dtype=torch.int32, device='cuda')
    s = torch.ones(1, 16, dtype=torch.float16, device='cuda')
    c = torch.empty(2, 16, dtype=torch.float16, device='cuda')
    with pytest.raises(ffi.BackendException, match='workspace') as e:
        f(a.data_ptr(), q.data_ptr(), s.data_ptr(), None, c.data_ptr(), 2, 16, 64, 64, None, 0, None)
    assert e.value.status == ffi.WORKSPACE_TOO_SMALL
    with pytest.raises(ValueError):
        w4a16_linear('x', 100, 64, 64)
    # the int8 path's counters at the head of a shared workspace stay untouched
    assert ffi.func('b200q_qlinear_f16_u4_workspace_bytes')(2, 16, 64, 64) > 65536 * 4
    w = torch.randn(4096, 4096, device='cuda').half() * 0.02
    wq, sc = hidet_b200.symmetric_quantize(w, 'int8', dims=0)
    x = torch.randn(2, 4096, device='cuda').half()
    before = hidet_b200.symmetric_quant_matmul(x, wq, sc)
    w4a16_linear('y', 64, 16, 64, with_zp=False)(a, q, s)
    assert torch.equal(hidet_b200.symmetric_quant_matmul(x, wq, sc), before)
    assert ffi.func('b200q_check_status')() == ffi.OK
