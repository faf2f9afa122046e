"""Measures the rcp.approx.ftz.f32 table the f16 oracle uses (run on a machine with a B200).

Compiles tests/golden/rcp_table.cu with nvcc, runs it and stores the 65536 results as
rcp_approx_ftz_f32_of_f16.npy (uint32) in the directory given by --out (default: this directory).

Usage: python tests/golden/make_rcp_table.py [--out DIR]
"""
import argparse
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument('--out', default=HERE)
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, 'rcp_table')
        raw = os.path.join(tmp, 'rcp.bin')
        subprocess.check_call(['nvcc', '-gencode', 'arch=compute_100a,code=sm_100a', '-O2', os.path.join(HERE, 'rcp_table.cu'), '-o', exe])
        subprocess.check_call([exe, raw])
        table = np.fromfile(raw, dtype=np.uint32)
    assert table.shape == (65536,)
    np.save(os.path.join(args.out, 'rcp_approx_ftz_f32_of_f16.npy'), table)
    # how far the instruction is from the correctly rounded reciprocal, for the record
    x = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    with np.errstate(all='ignore'):
        exact = (np.float32(1.0) / x).astype(np.float32)
    finite = np.isfinite(exact) & np.isfinite(x) & (x != 0)
    diff = table.astype(np.int64)[finite] - exact.view(np.uint32).astype(np.int64)[finite]
    print('entries that differ from the correctly rounded reciprocal: {} of {}, largest difference {} ulp'.format(
        int((diff != 0).sum()), int(finite.sum()), int(np.abs(diff).max())))
    return 0


if __name__ == '__main__':
    sys.exit(main())
