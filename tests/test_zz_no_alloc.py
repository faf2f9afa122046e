"""b200q_qlinear_f16_i8_static: the entry point for callers that cannot allocate scratch memory.

Some users of the library only ever hold device pointers and a stream (a compiled graph's launch
function, a plugin inside another runtime, a process with fully pre-partitioned device memory) and
therefore cannot give the kernel a workspace, nor call cudaMalloc.  For them the library carries a
fixed 512 KiB scratch array.  This test calls that entry point through the C ABI, on shapes that really
use the scratch, twice in a row, and compares with the regular entry point, which gets a
caller-allocated workspace.  Both run the same deterministic kernel, so the outputs must be identical.
"""
import pytest
import torch

import hidet_b200
from hidet_b200 import ffi

pytestmark = pytest.mark.gpu


def _problem(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(k, n, generator=g) * 0.02).to(torch.float16).cuda()
    wq, scale = hidet_b200.symmetric_quantize(w, 'int8', dims=0)
    a = torch.randn(m, k, generator=g).to(torch.float16).cuda()
    return a, wq, scale


def _static_call(a, wq, scale, out):
    m, k = a.shape
    n = wq.shape[1]
    ffi.func('b200q_qlinear_f16_i8_static')(a.data_ptr(), wq.data_ptr(), scale.data_ptr(), out.data_ptr(), m, n, k, ffi.LAYOUT_KN,
                                            torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize('m,n,k', [(4, 256, 16384), (8, 1024, 28672), (1, 4096, 4096), (64, 512, 1024)])
def test_static_entry_point_matches_the_regular_one_twice(m, n, k):
    a, wq, scale = _problem(m, n, k, seed=m + n)
    want = hidet_b200.symmetric_quant_matmul(a, wq, scale)
    for call in range(2):
        out = torch.full((m, n), float('nan'), dtype=torch.float16, device='cuda')
        _static_call(a, wq, scale, out)
        torch.cuda.synchronize()
        assert torch.equal(out, want), 'call {}: {} elements differ'.format(call, int((out != want).sum()))
    # a different problem in between must not disturb the next call (the array keeps old contents)
    a2, wq2, scale2 = _problem(8, 512, 8192, seed=99)
    out2 = torch.empty(8, 512, dtype=torch.float16, device='cuda')
    _static_call(a2, wq2, scale2, out2)
    assert torch.equal(out2, hidet_b200.symmetric_quant_matmul(a2, wq2, scale2))
    out = torch.empty(m, n, dtype=torch.float16, device='cuda')
    _static_call(a, wq, scale, out)
    assert torch.equal(out, want)
    assert ffi.func('b200q_check_status')() == ffi.OK


def test_static_entry_point_with_an_empty_sum_writes_zeros_like_the_regular_one():
    a = torch.zeros(3, 0, dtype=torch.float16, device='cuda')
    wq = torch.zeros(0, 64, dtype=torch.int8, device='cuda')
    scale = torch.ones(64, dtype=torch.float16, device='cuda')
    out = torch.full((3, 64), 5.0, dtype=torch.float16, device='cuda')
    ffi.func('b200q_qlinear_f16_i8_static')(0, 0, scale.data_ptr(), out.data_ptr(), 3, 64, 0, ffi.LAYOUT_KN, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert not out.any()


def test_static_entry_point_uses_scratch_on_these_shapes():
    ws = ffi.func('b200q_qlinear_workspace_bytes')
    limit = ffi.func('b200q_qlinear_static_scratch_bytes')()
    assert limit == 512 << 10
    assert 0 < ws(4, 256, 16384, ffi.LAYOUT_KN) <= limit
    assert 0 < ws(8, 1024, 28672, ffi.LAYOUT_KN) <= limit


def test_static_entry_point_refuses_what_does_not_fit():
    m, n, k = 32, 512, 28672
    assert ffi.func('b200q_qlinear_workspace_bytes')(m, n, k, ffi.LAYOUT_KN) > (512 << 10)
    a = torch.zeros(m, k, dtype=torch.float16, device='cuda')
    wq = torch.zeros(k, n, dtype=torch.int8, device='cuda')
    scale = torch.ones(n, dtype=torch.float16, device='cuda')
    out = torch.empty(m, n, dtype=torch.float16, device='cuda')
    with pytest.raises(ffi.BackendException, match='built-in scratch holds 524288') as e:
        _static_call(a, wq, scale, out)
    assert e.value.status == ffi.WORKSPACE_TOO_SMALL
    with pytest.raises(ffi.BackendException, match='16-byte aligned'):
        _static_call(a[:, :100].contiguous(), wq[:100, :20].contiguous(), scale[:20].contiguous(), out[:, :20].contiguous())
