"""Host logic of the column-parallel linear under gloo, world size 2, on CPU.

The kernels are CUDA-only, so each rank's output slice is produced by the CPU oracle here; what is
under test is the sharding arithmetic and the gather (rank-major all-gather, side-by-side placement)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, m: int, result_dir: str):
    sys.path.insert(0, ROOT)
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        import oracle
        from hidet_b200 import distributed as hd

        k, n = 256, 128
        rng = np.random.default_rng(7)  # every rank draws the full tensors and slices
        w = (rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)).astype(np.float16)
        a = rng.standard_normal((m, k), dtype=np.float32).astype(np.float16)
        wq_full, scale_full = oracle.symmetric_quantize(w, 'int8', 0)
        # quantizing the shard gives the shard of the quantized weight
        w_shard, _ = hd.shard_columns(torch.from_numpy(w), None, rank, world)
        wq_r, scale_r = oracle.symmetric_quantize(w_shard.numpy(), 'int8', 0)
        begin, end = hd.column_range(n, rank, world)
        assert np.array_equal(wq_r, wq_full[:, begin:end]) and np.array_equal(scale_r, scale_full[begin:end])
        wq_s, scale_s = hd.shard_columns(torch.from_numpy(wq_full), torch.from_numpy(scale_full), rank, world)
        assert np.array_equal(wq_s.numpy(), wq_r) and np.array_equal(scale_s.numpy(), scale_r)
        c_local = torch.from_numpy(oracle.symmetric_quant_matmul(a, wq_r, scale_r))
        # the reference op's layout: [nranks, *x.shape]
        y = hd.all_gather(c_local)
        assert tuple(y.shape) == (world, m, n // world) and torch.equal(y[rank], c_local)
        c = hd.gather_columns(c_local)
        want = torch.from_numpy(oracle.symmetric_quant_matmul(a, wq_full, scale_full))
        assert tuple(c.shape) == (m, n) and torch.equal(c, want)
        # batched activations keep their leading dims
        c3 = hd.gather_columns(c_local.reshape(1, m, n // world))
        assert tuple(c3.shape) == (1, m, n) and torch.equal(c3[0], want)
        with open(os.path.join(result_dir, 'ok{}'.format(rank)), 'w') as f:
            f.write('ok')
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('m', [1, 5])
def test_column_parallel_gather_world2(tmp_path, m):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), m, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(os.path.join(str(tmp_path), 'ok{}'.format(r))) for r in range(world))


def test_column_range_rejects_uneven_splits():
    from hidet_b200.distributed import column_range

    assert column_range(28672, 3, 8) == (10752, 14336)
    with pytest.raises(ValueError):
        column_range(100, 0, 8)
