"""Generates tests/golden/reference_cpu_*.npz by running the reference (hidet-org/hidet) itself.

Needs the reference checkout (its path in the environment variable HIDET_REFERENCE) and cmake, g++.
It only runs where the checkout exists; the fixtures it writes are committed so that the tests need
neither.  Nothing is written into the checkout: its runtime library is built out of tree, and its
python package is imported from a scratch copy (the package looks for its native libraries relative
to its own path, so it cannot be imported in place from a read-only tree).

The reference has no CPU implementation of float16 quantization (its generated x86 code for `half`
does not compile), so what runs here is its float32 x86 path: symmetric_quantize,
symmetric_dequantize, matmul, and the graph quantization pass (PassContext.set_precision('int8')).

Usage: python tests/golden/gen_reference_cpu.py [--scratch DIR]
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
import textwrap

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE = os.environ.get('HIDET_REFERENCE', '')


def prepare_reference(scratch: str) -> None:
    """Out-of-tree build of libhidet_runtime.so plus an importable scratch copy of python/hidet."""
    build = os.path.join(scratch, 'build')
    os.makedirs(build, exist_ok=True)
    if not os.path.exists(os.path.join(build, 'lib', 'libhidet_runtime.so')):
        subprocess.check_call(['cmake', REFERENCE, '-DCMAKE_BUILD_TYPE=Release'], cwd=build, stdout=subprocess.DEVNULL)
        subprocess.check_call(['make', '-j8'], cwd=build, stdout=subprocess.DEVNULL)
    pkg = os.path.join(scratch, 'python', 'hidet')
    if not os.path.exists(pkg):
        shutil.copytree(os.path.join(REFERENCE, 'python', 'hidet'), pkg)
    inc = os.path.join(scratch, 'include')
    if not os.path.exists(inc):
        os.symlink(os.path.join(REFERENCE, 'include'), inc)
    stubs = os.path.join(scratch, 'stubs')
    files = {
        # packages the reference imports unconditionally and this image lacks
        'tomlkit/__init__.py': '''
            class TOMLDocument(dict):
                def add(self, *a, **k): pass
            def document(): return TOMLDocument()
            def table(): return TOMLDocument()
            def comment(x): return x
            def nl(): return None
            def array(): return []
            def parse(s): return {}
            def dump(doc, f): f.write('')
            ''',
        'hip/__init__.py': 'from . import hip\n',
        'hip/hip.py': '''
            class _Dummy:
                def __init__(self, *a, **k): pass
                def __getattr__(self, n): return _Dummy()
                def __call__(self, *a, **k): return _Dummy()
            def __getattr__(name):
                return _Dummy
            ''',
        'nvtx/__init__.py': '''
            def annotate(*a, **k):
                def deco(f): return f
                return deco
            ''',
        'hidet-0.0.0.dist-info/METADATA': 'Metadata-Version: 2.1\nName: hidet\nVersion: 0.0.0\n',
    }
    for rel, text in files.items():
        path = os.path.join(stubs, rel)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, 'w') as f:
            f.write(textwrap.dedent(text).lstrip('\n'))
    sys.path[:0] = [os.path.join(scratch, 'python'), stubs]
    os.environ.setdefault('HOME', os.path.join(scratch, 'home'))


def import_reference(scratch: str):
    import hidet
    from hidet.drivers import utils as driver_utils
    from hidet.runtime import storage
    from hidet.runtime.device import Device

    hidet.option.cache_dir(os.path.join(scratch, 'cache'))
    # No GPU in the generating container: keep the reference off the CUDA driver.
    hidet.option.cuda.arch('sm_100')
    driver_utils.lazy_initialize_cuda._initialized = True
    cpu = Device('cpu')
    storage._device2pool.device2pool[cpu] = storage.MemoryPool(
        storage.CpuMemoryAPI(cpu), block_size=4096, max_reserve_size=512 * 1024**2)
    return hidet


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument('--scratch', default='/tmp/hidet_reference_scratch')
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(REFERENCE, 'python', 'hidet')):
        print('set HIDET_REFERENCE to a checkout of hidet-org/hidet', file=sys.stderr)
        return 2
    prepare_reference(args.scratch)
    hidet = import_reference(args.scratch)
    import torch

    def from_np(x):
        return hidet.from_torch(torch.from_numpy(np.ascontiguousarray(x)))

    rng = np.random.default_rng(20240607)

    # ---- 1. quantize / dequantize round trips: the shapes, dims and types of the reference's own test
    #         (tests/operators_core/test_symmetric_quant.py:19-26) plus a weight-like case and edge rows ----
    cases = {}
    specs = [
        ('t32_i8_last', (32, 32), 'int8', [-1], 1.0),
        ('t32_i8_first', (32, 32), 'int8', [0], 1.0),
        ('t64_i16_last', (64, 64), 'int16', [-1], 1.0),
        ('t64_i16_first', (64, 64), 'int16', [0], 1.0),
        ('w256x192_i8_first', (256, 192), 'int8', [0], 0.02),
        ('w96x200_i8_last', (96, 200), 'int8', [-1], 0.02),
        ('odd67x45_i8_first', (67, 45), 'int8', [0], 0.02),
    ]
    for name, shape, qt, dims, std in specs:
        w = (rng.standard_normal(shape) * std).astype(np.float32)
        if name.startswith('w256'):
            w[:, 3] = 0.0            # a column of zeros: scale 0, 0/0
            w[:, 5] = np.abs(w[:, 5])  # all positive
            w[7, 9] = 0.5            # an outlier that owns its column's scale
        wq, scale = hidet.ops.symmetric_quantize(from_np(w), qt, dims=dims)
        wd = hidet.ops.symmetric_dequantize(wq, scale, dims=dims)
        cases[name] = dict(w=w, wq=wq.numpy().copy(), scale=scale.numpy().copy(), wd=wd.numpy().copy(),
                           dims=np.array(dims), quant_type=qt)
    flat = {}
    for name, d in cases.items():
        for k, v in d.items():
            flat['{}/{}'.format(name, k)] = v
    np.savez_compressed(os.path.join(HERE, 'reference_cpu_quantize.npz'), **flat)

    # ---- 2. the CPU plumbing configuration at reduced size: quantize, dequantize, matmul, and the same
    #         through the graph pass ----
    K, N, M = 512, 384, 16
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    a = rng.standard_normal((M, K)).astype(np.float32)
    wq, scale = hidet.ops.symmetric_quantize(from_np(w), 'int8', dims=0)
    wd = hidet.ops.symmetric_dequantize(wq, scale, dims=0)
    c_eager = hidet.ops.matmul(from_np(a), wd)

    xs = hidet.symbol([M, K], dtype='float32', device='cpu')
    graph = hidet.trace_from(hidet.ops.matmul(xs, from_np(w)), xs)
    with hidet.graph.PassContext() as ctx:
        ctx.set_precision('int8')
        graph_q = hidet.graph.optimize(graph)
    c_graph = graph_q(from_np(a))
    op_names = [type(node).__name__ for node in graph_q.nodes]
    np.savez_compressed(
        os.path.join(HERE, 'reference_cpu_linear.npz'),
        w=w, a=a, wq=wq.numpy().copy(), scale=scale.numpy().copy(), wd=wd.numpy().copy(),
        c_eager=c_eager.numpy().copy(), c_graph=c_graph.numpy().copy(), graph_ops=np.array(op_names),
    )

    # ---- 3. full-size configuration (W fp32 [4096, 4096] ~ N(0, 0.02), A fp32 [16, 4096]): digests only ----
    rng_full = np.random.default_rng(4096)
    w = (rng_full.standard_normal((4096, 4096)) * 0.02).astype(np.float32)
    a = rng_full.standard_normal((16, 4096)).astype(np.float32)
    wq, scale = hidet.ops.symmetric_quantize(from_np(w), 'int8', dims=0)
    wd = hidet.ops.symmetric_dequantize(wq, scale, dims=0)
    c = hidet.ops.matmul(from_np(a), wd)
    wq_np, scale_np, c_np = wq.numpy().copy(), scale.numpy().copy(), c.numpy().copy()
    np.savez_compressed(
        os.path.join(HERE, 'reference_cpu_full_digest.npz'),
        seed=np.array(4096), w_sha256=np.array(sha(w)), a_sha256=np.array(sha(a)),
        wq_sha256=np.array(sha(wq_np)), scale=scale_np, c=c_np,
        wq_column_sums=wq_np.astype(np.int64).sum(axis=0), wq_row_sums=wq_np.astype(np.int64).sum(axis=1),
    )
    print('wrote fixtures to', HERE)
    print('graph ops after the int8 pass:', op_names)
    return 0


if __name__ == '__main__':
    sys.exit(main())
