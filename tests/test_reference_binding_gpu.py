"""The drop-in, exercised from the reference's side.

oracle/b200q_binding.py defines a task of the reference whose CUDA implementation is a `launch` that calls
b200q_qlinear_f16_i8 (stream and workspace from the reference's runtime, errors forwarded to
hidet_set_last_error).  oracle/build_ref.py lets the reference generate that module and compiles it with the
reference's flags against include/hidet_b200q.h and libhidet_b200q.so.  Here its `hidet_launch` is called on the
GPU the way the reference calls every compiled task (raw pointers, inputs then outputs), through the
reference's own runtime library, and compared with this repository's host layer bit for bit.
"""
import pytest
import torch

from conftest import seeded_activation, seeded_weight

import hidet_b200
from hidet_b200 import ffi
from oracle import ref_kernels

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_kernels.available(), reason='oracle/_ref has not been built')]


@pytest.fixture(scope='module')
def ref():
    r = ref_kernels.ReferenceKernels()
    if r.find('b200q_task', m=4, k=4096, n=4096) is None:
        pytest.skip('oracle/_ref holds no b200q task libraries')
    return r


@pytest.mark.parametrize('m,k,n', [(4, 4096, 4096), (16, 8192, 1024), (300, 1024, 768), (3, 100, 36)])
def test_reference_task_launch_reaches_the_library(ref, m, k, n):
    w = torch.from_numpy(seeded_weight(k, n, seed=k + n)).cuda()
    a = torch.from_numpy(seeded_activation(m, k, seed=m)).cuda()
    wq, scale = hidet_b200.symmetric_quantize(w, 'int8', dims=0)
    want = hidet_b200.symmetric_quant_matmul(a, wq, scale)
    name = ref.find('b200q_task', m=m, k=k, n=n)
    for _ in range(2):   # the second call reuses the runtime's workspace
        c = torch.full((m, n), float('nan'), dtype=torch.float16, device='cuda')
        ref.launch(name, a, wq, scale, c)
        assert torch.equal(c, want)
    assert ffi.func('b200q_check_status')() == ffi.OK


def test_library_errors_surface_through_the_reference_runtime(ref):
    a = torch.zeros(4, 4096, dtype=torch.float16, device='cuda')
    wq = torch.zeros(4096, 4096, dtype=torch.int8, device='cuda')
    scale = torch.ones(4096, dtype=torch.float16, device='cuda')
    name = ref.find('b200q_task', m=4, k=4096, n=4096)
    with pytest.raises(RuntimeError, match='null output or scale pointer'):
        ref.launch_pointers(name, a.data_ptr(), wq.data_ptr(), scale.data_ptr(), 0)
    # read and cleared: the next good call raises nothing
    c = torch.empty(4, 4096, dtype=torch.float16, device='cuda')
    ref.launch(name, a, wq, scale, c)
    assert not c.any()
