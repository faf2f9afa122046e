"""The prebuilt libraries of the reference's own kernels (oracle/_ref) load and export what the harness binds.
No compute: that needs a GPU (tests/test_reference_kernels_gpu.py)."""
import ctypes
import os

import pytest

from oracle import build_ref, ref_kernels

pytestmark = pytest.mark.skipif(not ref_kernels.available(), reason='oracle/_ref has not been built')


def test_manifest_lists_every_case_of_the_recipe():
    import json

    manifest = json.load(open(os.path.join(ref_kernels.REF_DIR, 'manifest.json')))
    assert [c['name'] for c in manifest['cases']] == [name for name, _, _ in build_ref.CASES]
    for case in manifest['cases']:
        assert os.path.exists(os.path.join(ref_kernels.REF_DIR, case['file']))


def test_libraries_load_and_export_the_launch_function():
    runtime = ctypes.CDLL(os.path.join(ref_kernels.REF_DIR, 'libhidet_runtime.so'), mode=ctypes.RTLD_GLOBAL)
    for symbol in ('register_callback', 'set_cuda_stream', 'use_torch_cuda_stream', 'request_cuda_workspace', 'hidet_get_last_error'):
        assert getattr(runtime, symbol)
    import torch  # noqa: F401  (brings the CUDA runtime library the case libraries link against)

    for name, _, _ in build_ref.CASES:
        lib = ctypes.CDLL(os.path.join(ref_kernels.REF_DIR, name + '.so'))
        assert lib.hidet_launch
