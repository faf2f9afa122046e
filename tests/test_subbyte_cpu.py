"""The 4-bit weight oracle (oracle/subbyte.py) against hand-written bytes and the reference's own check (no GPU)."""
import numpy as np

from oracle import subbyte


def test_nibble_order_is_the_reference_s_subbyte_storage():
    # element i of a row: (byte[i / 2] >> (4 * (i % 2))) & 15  (python/hidet/transforms/lower_integer_subbyte.py:103-113)
    packed = subbyte.pack_u4(np.array([[1, 2, 3, 4, 15, 0, 9, 10]], dtype=np.float16))
    assert packed.tolist() == [[0x21, 0x43, 0x0F, 0xA9]]
    assert subbyte.unpack_u4(packed).tolist() == [[1, 2, 3, 4, 15, 0, 9, 10]]
    # eight codes per int32 word, code i in bits 4 i .. 4 i + 3
    assert packed.view(np.uint32).tolist() == [[0xA90F4321]]
    # C conversion to int, low four bits: 17.9 -> 17 -> 1, -1.0 -> -1 -> 15
    assert subbyte.unpack_u4(subbyte.pack_u4(np.array([[17.9, -1.0]]))).tolist() == [[1, 15]]


def test_linear_equals_the_exact_result_on_the_reference_s_test_data():
    """tests/cute_kernel/test_quant_linear.py:36-85: small integers everywhere, so `a @ (scale * (b - zeros))` is exact
    in any float type and every order of summation gives the same number."""
    rng = np.random.default_rng(0)
    m, n, k, g = 3, 64, 256, 128
    a = rng.integers(-3, 3, (m, k)).astype(np.float16)
    b = rng.integers(0, 3, (k, n))
    scale = rng.integers(0, 2, (k // g, n)).astype(np.float16)
    zeros = rng.integers(0, 3, (k // g, n)).astype(np.float16)
    packed = subbyte.pack_u4(b.astype(np.float16))
    for with_zp in (True, False):
        w = np.zeros((k, n), dtype=np.int64)
        for kk in range(k):
            w[kk] = scale[kk // g].astype(np.int64) * (b[kk] - (zeros[kk // g].astype(np.int64) if with_zp else 0))
        want = a.astype(np.int64) @ w
        for f16_steps in (False, True):
            got = subbyte.w4a16_linear(a, packed, scale, zeros if with_zp else None, g, f16_steps)
            assert np.array_equal(got, want.astype(np.float64))
