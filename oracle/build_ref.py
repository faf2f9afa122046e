"""Builds oracle/_ref/: the reference's own CUDA kernels for this path, compiled for sm_100a.

Test infrastructure only.  The reference (hidet-org/hidet) generates one CUDA source per task and compiles
it with nvcc at run time.  This recipe does the same ahead of time, where a checkout of the reference is at
hand and no GPU is needed:

  1. its small C++ runtime (ten files under src/hidet/runtime, named in its CMakeLists.txt) is compiled
     with g++ directly from where the files lie -> oracle/_ref/libhidet_runtime.so;
  2. its Python package is imported from a scratch copy and asked to generate the CUDA source of the
     quantize / dequantize / quantized-matmul tasks at the listed shapes (python/hidet/graph/ops/quant/
     symmetric.py:23-61, matmul.py:24-74, matmul_f16_i8.py:30-93), exactly as its own build does
     (python/hidet/drivers/build_module.py, python/hidet/backend/codegen.py);
  3. each source is compiled with the flags of python/hidet/backend/build.py:152-200 (-O3, -std=c++11,
     -ftz=true, -prec-div=false, arch sm_100a) -> oracle/_ref/<case>.so exporting `hidet_launch`.

Only binaries and a manifest are written under oracle/_ref/ (git-ignored); generated sources stay in the
scratch directory.  tests/test_reference_kernels_gpu.py runs these kernels on the GPU beside this
repository's and compares bits.

Usage: python oracle/build_ref.py [--scratch DIR] [--force]
The checkout is taken from the environment variable HIDET_REFERENCE, else from a directory `reference`
beside the repository.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, '_ref')

INCLUDE_DIR = os.path.join(ROOT, 'include')
LIBRARY_DIR = os.path.join(ROOT, 'hidet_b200', 'lib')

RUNTIME_SOURCES = [
    'src/hidet/runtime/cuda/context.cpp', 'src/hidet/runtime/cuda/cublas.cpp', 'src/hidet/runtime/cuda/cudnn.cpp',
    'src/hidet/runtime/cuda/cuda.cpp', 'src/hidet/runtime/hip/context.cpp', 'src/hidet/runtime/cpu/context.cpp',
    'src/hidet/runtime/callbacks.cpp', 'src/hidet/runtime/logging.cpp', 'src/hidet/runtime/symbols.cpp',
    'src/hidet/runtime/int_fastdiv.cpp',
]

# (case name, task kind, parameters).  Shapes: the decode projections of the benchmark, the reference's own
# test shapes (tests/operators_core/test_symmetric_quant.py:19-26) and ragged ones.
CASES = [
    ('quant_f16_d0_4096x4096', 'quantize', {'rows': 4096, 'cols': 4096, 'dims': 0}),
    ('quant_f16_d0_4096x11008', 'quantize', {'rows': 4096, 'cols': 11008, 'dims': 0}),
    ('quant_f16_d0_200x48', 'quantize', {'rows': 200, 'cols': 48, 'dims': 0}),
    ('quant_f16_d0_77x130', 'quantize', {'rows': 77, 'cols': 130, 'dims': 0}),
    ('quant_f16_d1_512x384', 'quantize', {'rows': 512, 'cols': 384, 'dims': -1}),
    ('quant_f16_d1_4096x4096', 'quantize', {'rows': 4096, 'cols': 4096, 'dims': -1}),
    ('dequant_f16_d0_4096x4096', 'dequantize', {'rows': 4096, 'cols': 4096, 'dims': 0}),
    ('dequant_f16_d0_200x48', 'dequantize', {'rows': 200, 'cols': 48, 'dims': 0}),
    ('qmm_f16_i8_16x4096x4096', 'matmul_f16_i8', {'m': 16, 'k': 4096, 'n': 4096}),
    ('qmm_f16_i8_1x4096x11008', 'matmul_f16_i8', {'m': 1, 'k': 4096, 'n': 11008}),
    ('qmm_generic_4x512x256', 'matmul_generic', {'m': 4, 'k': 512, 'n': 256}),
    # the other types the reference's own tests run (tests/operators_core/test_symmetric_quant.py:19-26,
    # tests/operators_core/test_quantization.py:21-36): int16 codes, bfloat16 weights
    ('quant_f16_i16_d0_200x48', 'quantize', {'rows': 200, 'cols': 48, 'dims': 0, 'qtype': 'int16'}),
    ('quant_f16_i16_d1_512x384', 'quantize', {'rows': 512, 'cols': 384, 'dims': -1, 'qtype': 'int16'}),
    ('quant_bf16_d0_200x48', 'quantize', {'rows': 200, 'cols': 48, 'dims': 0, 'wtype': 'bfloat16'}),
    ('quant_bf16_d1_512x384', 'quantize', {'rows': 512, 'cols': 384, 'dims': -1, 'wtype': 'bfloat16'}),
    ('quant_bf16_d0_4096x4096', 'quantize', {'rows': 4096, 'cols': 4096, 'dims': 0, 'wtype': 'bfloat16'}),
    ('dequant_f16_i16_d0_200x48', 'dequantize', {'rows': 200, 'cols': 48, 'dims': 0, 'qtype': 'int16'}),
    ('dequant_bf16_d0_200x48', 'dequantize', {'rows': 200, 'cols': 48, 'dims': 0, 'wtype': 'bfloat16'}),
    # The drop-in itself: a task of the reference whose CUDA implementation is a `launch` that calls this
    # repository's library (b200q_task below), generated, compiled and linked the reference's way.
    ('b200q_task_4x4096x4096', 'b200q_task', {'m': 4, 'k': 4096, 'n': 4096}),
    ('b200q_task_16x8192x1024', 'b200q_task', {'m': 16, 'k': 8192, 'n': 1024}),
    ('b200q_task_300x1024x768', 'b200q_task', {'m': 300, 'k': 1024, 'n': 768}),
    ('b200q_task_3x100x36', 'b200q_task', {'m': 3, 'k': 100, 'n': 36}),
]



def reference_root() -> str:
    ref = os.environ.get('HIDET_REFERENCE') or os.path.join(os.path.dirname(ROOT), 'reference')
    return ref if os.path.isdir(os.path.join(ref, 'python', 'hidet')) else ''


def recipe_digest(ref: str) -> str:
    h = hashlib.sha256()
    h.update(open(os.path.abspath(__file__), 'rb').read())
    for rel in RUNTIME_SOURCES + ['python/hidet/graph/ops/quant/symmetric.py', 'python/hidet/graph/ops/quant/matmul.py',
                                  'python/hidet/graph/ops/quant/matmul_f16_i8.py', 'python/hidet/backend/build.py']:
        h.update(open(os.path.join(ref, rel), 'rb').read())
    return h.hexdigest()


def build_runtime(ref: str, scratch: str) -> None:
    """g++ on the reference's runtime sources, where they lie; a copy where its Python package looks for it."""
    lib_dir = os.path.join(scratch, 'build', 'lib')
    os.makedirs(lib_dir, exist_ok=True)
    os.makedirs(OUT, exist_ok=True)
    runtime = os.path.join(OUT, 'libhidet_runtime.so')
    cmd = ['g++', '-O2', '-std=c++17', '-fPIC', '-shared', '-I' + os.path.join(ref, 'include'), '-I/usr/local/cuda/include']
    cmd += [os.path.join(ref, s) for s in RUNTIME_SOURCES] + ['-o', runtime, '-ldl']
    subprocess.check_call(cmd)
    shutil.copy(runtime, os.path.join(lib_dir, 'libhidet_runtime.so'))
    subprocess.check_call(['g++', '-O2', '-fPIC', '-shared', os.path.join(ref, 'src', 'hidet', 'empty.cpp'), '-o', os.path.join(lib_dir, 'libhidet.so'),
                           '-L' + lib_dir, '-Wl,--no-as-needed', '-lhidet_runtime', '-Wl,-rpath,$ORIGIN'])


def generate_sources(ref: str, scratch: str) -> dict:
    """Imports the reference from the scratch copy and lets it write the CUDA source of every case."""
    os.environ['HIDET_REFERENCE'] = ref
    sys.path.insert(0, os.path.join(ROOT, 'tests', 'golden'))
    sys.path.insert(0, HERE)
    import gen_reference_cpu as helper   # scratch copy of the package, stand-ins for packages this image lacks

    helper.REFERENCE = ref
    helper.prepare_reference(scratch)
    hidet = helper.import_reference(scratch)
    from hidet.backend import codegen
    from hidet.drivers.build_module import lower_ir_module
    from hidet.graph.ops.quant.matmul import SymmetricQuantizedMatmulTask
    from hidet.graph.ops.quant.matmul_f16_i8 import SymmetricQuantizedMatmulF16I8Task
    from hidet.graph.ops.quant.symmetric import SymmetricDeQuantizationTask, SymmetricQuantizationTask
    from hidet.ir import dtypes
    from hidet.ir.compute import tensor_input
    from hidet.ir.target import Target

    hidet.option.cuda.arch('sm_100')
    target = Target.from_string('cuda')
    sources = {}
    for name, kind, p in CASES:
        wtype, qtype = p.get('wtype', 'float16'), p.get('qtype', 'int8')
        if kind == 'quantize':
            task = SymmetricQuantizationTask(tensor_input('w', wtype, [p['rows'], p['cols']]), getattr(dtypes, qtype), dims=p['dims'])
        elif kind == 'dequantize':
            scale_len = p['cols'] if p['dims'] == 0 else p['rows']
            task = SymmetricDeQuantizationTask(tensor_input('wq', qtype, [p['rows'], p['cols']]), tensor_input('scale', wtype, [scale_len]), dims=p['dims'])
        elif kind == 'b200q_task':
            import b200q_binding

            task = b200q_binding.b200q_task(hidet, tensor_input('a', 'float16', [p['m'], p['k']]), tensor_input('b', 'int8', [p['k'], p['n']]),
                              tensor_input('scale', 'float16', [p['n']]))
        elif kind == 'matmul_f16_i8':
            task = SymmetricQuantizedMatmulF16I8Task(tensor_input('a', 'float16', [p['m'], p['k']]), tensor_input('b', 'int8', [p['k'], p['n']]),
                                                     tensor_input('scale', 'float16', [p['n']]), 1)
        else:
            task = SymmetricQuantizedMatmulTask(tensor_input('a', 'float16', [p['m'], p['k']]), tensor_input('b', 'int8', [p['k'], p['n']]),
                                                tensor_input('scale', 'float16', [p['n']]))
        work = os.path.join(scratch, 'wd', name)
        os.makedirs(work, exist_ok=True)
        modules = task.implement('cuda', work)
        # the first candidate of the schedule space (the reference picks among them by timing on a GPU)
        module = lower_ir_module(modules[0], work, target)
        src = os.path.join(work, 'source.cu')
        codegen(module, src_out_path=src, target=target)
        sources[name] = src
    return sources


def compile_case(ref: str, src: str, out: str, binding: bool = False) -> None:
    extra = []
    if binding:  # what the reference's build adds for ir_module.include_dirs / linking_dirs / linking_libs
        extra = ['-I' + INCLUDE_DIR, '-L' + LIBRARY_DIR, '-l:libhidet_b200q.so', '-Xlinker', '-rpath,$ORIGIN/../../hidet_b200/lib']
    cmd = ['nvcc', *extra, '-I' + os.path.join(ref, 'include'), '-L' + OUT, '-O3', '-Xcompiler', '-fPIC,-m64,-O3,-funroll-loops,-ffast-math', '-std=c++11',
           '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-ftz=true', '-prec-div=false', '-lhidet_runtime', '--cudart', 'shared',
           '--diag-suppress', '177', '--diag-suppress', '179', '--diag-suppress', '39', '-Xlinker', '-rpath,$ORIGIN', '--shared', src, '-o', out]
    subprocess.check_call(cmd, stdout=subprocess.DEVNULL)


def build(scratch: str = '', force: bool = False) -> bool:
    """Returns True when oracle/_ref/ is complete afterwards, False when no checkout of the reference is at hand."""
    ref = reference_root()
    if not ref:
        return os.path.exists(os.path.join(OUT, 'manifest.json'))
    digest = recipe_digest(ref)
    manifest_path = os.path.join(OUT, 'manifest.json')
    if not force and os.path.exists(manifest_path):
        old = json.load(open(manifest_path))
        if old.get('digest') == digest and all(os.path.exists(os.path.join(OUT, c['file'])) for c in old['cases']):
            return True
    scratch = scratch or os.path.join(tempfile.gettempdir(), 'hidet_b200_ref_build')
    build_runtime(ref, scratch)
    # the generation imports the reference, which must not leak into the calling process: run it apart
    listing = os.path.join(scratch, 'sources.json')
    subprocess.check_call([sys.executable, os.path.abspath(__file__), '--generate-only', '--scratch', scratch, '--listing', listing],
                          env=dict(os.environ, HIDET_REFERENCE=ref))
    sources = json.load(open(listing))
    cases = []
    for name, kind, p in CASES:
        compile_case(ref, sources[name], os.path.join(OUT, name + '.so'), binding=(kind == 'b200q_task'))
        if kind == 'b200q_task' and name == 'b200q_task_4x4096x4096':
            shutil.copy(sources[name], os.path.join(OUT, 'b200q_task_source.cu.txt'))   # quoted in the integration notes
        cases.append({'name': name, 'kind': kind, 'file': name + '.so', **p})
    json.dump({'digest': digest, 'runtime': 'libhidet_runtime.so', 'cases': cases}, open(manifest_path, 'w'), indent=1)
    return True


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument('--scratch', default='')
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--generate-only', action='store_true', help=argparse.SUPPRESS)
    ap.add_argument('--listing', default='', help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.generate_only:
        json.dump(generate_sources(reference_root(), args.scratch), open(args.listing, 'w'))
        return 0
    if not reference_root():
        print('no checkout of the reference found (set HIDET_REFERENCE)', file=sys.stderr)
        return 2
    build(args.scratch, args.force)
    print('built', OUT)
    return 0


if __name__ == '__main__':
    sys.exit(main())
