"""The CPU oracle against outputs of the reference itself (tests/golden/reference_cpu_*.npz, written
by tests/golden/gen_reference_cpu.py from the reference's compiled x86 tasks)."""
import hashlib
import os

import numpy as np
import pytest

from conftest import GOLDEN

import oracle


def _cases():
    q = np.load(os.path.join(GOLDEN, 'reference_cpu_quantize.npz'))
    names = sorted({k.split('/')[0] for k in q.files})
    return q, names


def test_quantize_matches_reference_cpu_vectors():
    q, names = _cases()
    assert len(names) >= 7
    for name in names:
        w = q[name + '/w']
        dims = q[name + '/dims'].tolist()
        qt = str(q[name + '/quant_type'])
        wq, scale = oracle.symmetric_quantize(w, qt, dims, x86_fast_math=True)
        # scales: bit-exact
        assert np.array_equal(scale.view(np.uint32), q[name + '/scale'].view(np.uint32)), name
        diff = wq.astype(np.int64) - q[name + '/wq'].astype(np.int64)
        if qt == 'int8':
            # int8 codes: bit-exact on every vector
            assert not diff.any(), name
        else:
            # int16 codes: the reference's -ffast-math build divides through a reciprocal estimate, which
            # moves a quotient that sits on a rounding boundary by one step in rare elements
            assert np.abs(diff).max() <= 1 and (diff != 0).mean() < 2e-3, name


def test_ieee_and_fast_math_scales_differ_by_at_most_one_ulp():
    q, names = _cases()
    for name in names:
        w = q[name + '/w']
        dims = q[name + '/dims'].tolist()
        _, s_ieee = oracle.symmetric_quantize(w, str(q[name + '/quant_type']), dims, x86_fast_math=False)
        d = s_ieee.view(np.uint32).astype(np.int64) - q[name + '/scale'].view(np.uint32).astype(np.int64)
        assert np.abs(d).max() <= 1, name


def test_dequantize_matches_reference_cpu_vectors():
    q, names = _cases()
    for name in names:
        wd = oracle.symmetric_dequantize(q[name + '/wq'], q[name + '/scale'], q[name + '/dims'].tolist())
        assert np.array_equal(wd.view(np.uint32), q[name + '/wd'].view(np.uint32)), name


def test_round_trip_tolerance_of_the_reference_test():
    # tests/operators_core/test_symmetric_quant.py:26 accepts atol = rtol = 1e-1
    q, names = _cases()
    for name in names:
        w = q[name + '/w']
        dims = q[name + '/dims'].tolist()
        wq, scale = oracle.symmetric_quantize(w, str(q[name + '/quant_type']), dims)
        wd = oracle.symmetric_dequantize(wq, scale, dims)
        finite = np.isfinite(wd)  # an all-zero column dequantizes to NaN in the reference as well
        assert np.allclose(wd[finite], w[finite], atol=1e-1, rtol=1e-1), name


def test_zero_column_behaves_like_the_reference():
    q, _ = _cases()
    name = 'w256x192_i8_first'
    wq, scale = oracle.symmetric_quantize(q[name + '/w'], 'int8', [0], x86_fast_math=True)
    assert scale[3] == 0 and np.array_equal(wq[:, 3], q[name + '/wq'][:, 3])


def test_linear_plumbing_configuration():
    l = np.load(os.path.join(GOLDEN, 'reference_cpu_linear.npz'))
    wq, scale = oracle.symmetric_quantize(l['w'], 'int8', 0, x86_fast_math=True)
    assert np.array_equal(wq, l['wq'])
    assert np.array_equal(scale.view(np.uint32), l['scale'].view(np.uint32))
    wd = oracle.symmetric_dequantize(l['wq'], l['scale'], 0)
    assert np.array_equal(wd.view(np.uint32), l['wd'].view(np.uint32))
    ref_max = np.abs(l['c_eager']).max()
    # same serial loop; the reference's build is -ffast-math, so sums may be reassociated
    c = oracle.matmul_f32(l['a'], l['wd'])
    assert np.abs(c - l['c_eager']).max() <= 1e-5 * ref_max
    c_q = oracle.symmetric_quant_matmul(l['a'], l['wq'], l['scale'])
    assert np.abs(c_q - l['c_graph']).max() <= 1e-5 * ref_max
    # the quantization pass really rewrote the matmul (one fused operator is left)
    assert list(l['graph_ops']) == ['FusedOperator']


def test_full_size_configuration_digests():
    d = np.load(os.path.join(GOLDEN, 'reference_cpu_full_digest.npz'))
    rng = np.random.default_rng(int(d['seed']))
    w = (rng.standard_normal((4096, 4096)) * 0.02).astype(np.float32)
    a = rng.standard_normal((16, 4096)).astype(np.float32)
    sha = lambda x: hashlib.sha256(np.ascontiguousarray(x).tobytes()).hexdigest()
    if sha(w) != str(d['w_sha256']) or sha(a) != str(d['a_sha256']):
        pytest.skip('this numpy draws different numbers from the seed than the one the digests were made with')
    wq, scale = oracle.symmetric_quantize(w, 'int8', 0, x86_fast_math=True)
    assert np.array_equal(scale.view(np.uint32), d['scale'].view(np.uint32))
    # 16.7 M codes; the reference's reciprocal-estimate division moves about one in a million by one step
    col = np.abs(wq.astype(np.int64).sum(0) - d['wq_column_sums']).sum()
    row = np.abs(wq.astype(np.int64).sum(1) - d['wq_row_sums']).sum()
    assert col <= 32 and row <= 32
    c = oracle.symmetric_quant_matmul(a, wq, scale)
    assert np.abs(c - d['c']).max() <= 1e-3 * np.abs(d['c']).max()


def test_half_conversions_are_ieee():
    lib = oracle.load()
    bits = np.arange(65536, dtype=np.uint16)
    ref = bits.view(np.float16).astype(np.float32)
    for h in range(0, 65536, 7):
        v = np.float32(lib.oracle_half_to_float(h))
        assert (np.isnan(v) and np.isnan(ref[h])) or v.view(np.uint32) == ref[h].view(np.uint32)
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.standard_normal(3000).astype(np.float32) * s for s in (1e-7, 1e-5, 1e-3, 1.0, 300.0, 70000.0)])
    with np.errstate(over='ignore'):
        want = x.astype(np.float16).view(np.uint16)
    got = np.array([lib.oracle_float_to_half(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(got, want)


def test_f16_quantize_properties():
    # the f16 arithmetic has no reference vectors (see quant_oracle.c); check what must hold anyway
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((128, 96)) * 0.02).astype(np.float16)
    for dims in (0, -1):
        wq, scale = oracle.symmetric_quantize(w, 'int8', dims)
        amax = np.abs(w).max(axis=0 if dims == 0 else 1)
        # scale = amax / 127 to within one half ulp of the approximate division
        assert np.allclose(scale.astype(np.float32), amax.astype(np.float32) / 127, rtol=2e-3)
        assert np.abs(wq.astype(np.int32)).max() == 127
        wd = oracle.symmetric_dequantize(wq, scale, dims)
        assert np.allclose(wd.astype(np.float32), w.astype(np.float32), atol=float(scale.max()), rtol=0)
    # quantize-then-slice == slice-then-quantize for per-column scales: what column sharding relies on
    wq_full, sc_full = oracle.symmetric_quantize(w, 'int8', 0)
    wq_part, sc_part = oracle.symmetric_quantize(np.ascontiguousarray(w[:, 32:64]), 'int8', 0)
    assert np.array_equal(wq_full[:, 32:64], wq_part) and np.array_equal(sc_full[32:64], sc_part)
