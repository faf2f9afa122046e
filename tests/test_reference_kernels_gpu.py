"""This repository's kernels and the CPU oracle against the reference's OWN CUDA kernels on the same GPU.

oracle/build_ref.py lets the reference generate the CUDA source of its quantize / dequantize / quantized-matmul
tasks and compiles it for sm_100a with the reference's flags (oracle/_ref/, prebuilt where a checkout of the
reference is at hand; the libraries travel, the checkout does not).  Here those kernels run beside ours on the same
seeded inputs: int8 codes, scales and dequantized values must agree bit for bit, matmul outputs within the
tolerance the benchmark specification sets (max |err| <= 1e-2 max |ref|; the reference's tensor-core kernel
accumulates in float16, so it is itself only that close to the exact sum).
"""
import numpy as np
import pytest
import torch

from conftest import seeded_activation, seeded_weight

import hidet_b200
import oracle
from oracle import ref_kernels

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_kernels.available(), reason='oracle/_ref has not been built')]


@pytest.fixture(scope='module')
def ref():
    return ref_kernels.ReferenceKernels()


def adversarial(rows, cols, seed):
    """Seeded weight with the columns / rows that stress the arithmetic: zeros (0/0), negative zeros, subnormals,
    the largest half, an outlier, a scale where the half division takes its correction step, exact ties."""
    w = seeded_weight(rows, cols, seed=seed)
    w[:, 0] = 0.0
    w[:, 1] = np.float16(-0.0)
    w[:, 2] = np.float16(6e-8)
    w[:, 3] = np.float16(65504.0)
    w[rows // 2, 4] = np.float16(30000.0)
    w[:, 5] = np.float16(1e-3)
    w[:, 6] = (np.arange(rows) % 7 - 3).astype(np.float16)
    w[1, :] = 0.0
    w[2, :] = (np.arange(cols) % 5 - 2).astype(np.float16) * np.float16(0.5)
    return w


def bits(t):
    return t.view(torch.int16)


@pytest.mark.parametrize('rows,cols,dims,kind', [
    (4096, 4096, 0, 'seeded'), (4096, 11008, 0, 'seeded'), (200, 48, 0, 'seeded'), (200, 48, 0, 'adversarial'),
    (77, 130, 0, 'seeded'), (77, 130, 0, 'adversarial'), (512, 384, -1, 'seeded'), (512, 384, -1, 'adversarial'),
    (4096, 4096, -1, 'seeded'),
])
def test_quantize_matches_the_reference_kernels_bit_for_bit(ref, rows, cols, dims, kind):
    w_np = adversarial(rows, cols, seed=rows + cols) if kind == 'adversarial' else seeded_weight(rows, cols, seed=rows + cols)
    w = torch.from_numpy(w_np).cuda()
    wq_ref, scale_ref = ref.symmetric_quantize(w, dims)
    wq, scale = hidet_b200.symmetric_quantize(w, 'int8', dims=dims)
    assert torch.equal(bits(scale), bits(scale_ref)), '{} scale words differ'.format(int((bits(scale) != bits(scale_ref)).sum()))
    assert torch.equal(wq, wq_ref), '{} of {} codes differ'.format(int((wq != wq_ref).sum()), wq.numel())
    if rows * cols <= 512 * 384:
        # the CPU oracle, pinned against the reference's kernels as run on this GPU
        wq_o, scale_o = oracle.symmetric_quantize(w_np, 'int8', dims)
        assert np.array_equal(scale_o.view(np.int16), bits(scale_ref).cpu().numpy())
        assert np.array_equal(wq_o, wq_ref.cpu().numpy())


@pytest.mark.parametrize('rows,cols', [(4096, 4096), (200, 48)])
def test_dequantize_matches_the_reference_kernels_bit_for_bit(ref, rows, cols):
    w = torch.from_numpy(seeded_weight(rows, cols, seed=5)).cuda()
    wq, scale = hidet_b200.symmetric_quantize(w, 'int8', dims=0)
    want = ref.symmetric_dequantize(wq, scale, 0)
    got = hidet_b200.symmetric_dequantize(wq, scale, dims=0)
    assert torch.equal(bits(got), bits(want))
    if rows * cols <= 512 * 384:
        got_o = oracle.symmetric_dequantize(wq.cpu().numpy(), scale.cpu().numpy(), 0)
        assert np.array_equal(got_o.view(np.int16), bits(want).cpu().numpy())


@pytest.mark.parametrize('rows,cols,dims,wtype,qtype,kind', [
    (200, 48, 0, 'float16', 'int16', 'seeded'), (200, 48, 0, 'float16', 'int16', 'adversarial'), (512, 384, -1, 'float16', 'int16', 'seeded'),
    (200, 48, 0, 'bfloat16', 'int8', 'seeded'), (200, 48, 0, 'bfloat16', 'int8', 'adversarial'), (512, 384, -1, 'bfloat16', 'int8', 'seeded'),
    (4096, 4096, 0, 'bfloat16', 'int8', 'seeded'),
])
def test_int16_codes_and_bfloat16_weights_match_the_reference_kernels_bit_for_bit(ref, rows, cols, dims, wtype, qtype, kind):
    """The other types the reference's tests run (tests/operators_core/test_symmetric_quant.py:19-26)."""
    w_np = adversarial(rows, cols, seed=rows + cols) if kind == 'adversarial' else seeded_weight(rows, cols, seed=rows + cols)
    w = torch.from_numpy(w_np).cuda().to(getattr(torch, wtype))
    wq_ref, scale_ref = ref.symmetric_quantize(w, dims, qtype)
    wq, scale = hidet_b200.symmetric_quantize(w, qtype, dims=dims)
    assert wq.dtype == wq_ref.dtype and scale.dtype == scale_ref.dtype
    assert torch.equal(bits(scale), bits(scale_ref)), '{} scale words differ'.format(int((bits(scale) != bits(scale_ref)).sum()))
    assert torch.equal(wq, wq_ref), '{} of {} codes differ'.format(int((wq != wq_ref).sum()), wq.numel())
    if (rows, cols, dims) == (200, 48, 0):
        want = ref.symmetric_dequantize(wq, scale, 0)
        got = hidet_b200.symmetric_dequantize(wq, scale, dims=0)
        assert torch.equal(bits(got), bits(want))


@pytest.mark.parametrize('m,k,n,kind', [(16, 4096, 4096, 'matmul_f16_i8'), (1, 4096, 11008, 'matmul_f16_i8'), (4, 512, 256, 'matmul_generic')])
def test_quantized_matmul_is_within_tolerance_of_the_reference_kernels(ref, m, k, n, kind):
    w = torch.from_numpy(seeded_weight(k, n, seed=k + n)).cuda()
    a = torch.from_numpy(seeded_activation(m, k, seed=m)).cuda()
    wq, scale = hidet_b200.symmetric_quantize(w, 'int8', dims=0)
    want = ref.quant_matmul(a, wq, scale, kind).float()
    got = hidet_b200.symmetric_quant_matmul(a, wq, scale).float()
    exact = (a.double() @ (wq.double() * scale.double())).float()
    top = exact.abs().max()
    assert torch.isfinite(want).all()
    assert (got - want).abs().max() <= 1e-2 * top
    # ours sums in float32 and rounds once: it is closer to the exact sum than the reference's float16 sums are
    assert (got - exact).abs().max() <= 1e-3 * top
    assert (got - exact).abs().max() <= (want - exact).abs().max() + 1e-3 * top
