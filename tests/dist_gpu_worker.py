"""Worker of tests/test_distributed_gpu.py (one process per GPU, started by torch.distributed.run):
checks the column-parallel quantized linear on real GPUs against the single-GPU result."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main() -> int:
    import hidet_b200
    from hidet_b200.distributed import ColumnParallelQuantLinear, column_range

    os.environ.setdefault('TORCH_SYMM_MEM_DISABLE_MULTICAST', '1')   # plain peer mappings only
    rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
    local = int(os.environ.get('LOCAL_RANK', rank))
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    dist.init_process_group('nccl', device_id=device)
    try:
        for k, n in ((1024, 2048), (8192, 3584 * world if world <= 2 else 1792 * world)):
            gen = torch.Generator(device=device).manual_seed(11)
            w = (torch.randn(k, n, generator=gen, device=device) * 0.02).half()
            wq_full, scale_full = hidet_b200.symmetric_quantize(w, 'int8', dims=0)
            begin, end = column_range(n, rank, world)
            for gather in ('nccl', 'p2p'):
                layer = ColumnParallelQuantLinear.from_weight_shard(w[:, begin:end].contiguous(), gather=gather)
                assert torch.equal(layer.wq, wq_full[:, begin:end]) and torch.equal(layer.scale, scale_full[begin:end])
                for m in (1, 16, 40, 300, 1100):
                    x = torch.randn(m, k, generator=gen, device=device).half()
                    # The split of K over CTAs depends on the width, so a shard's sums are taken in another
                    # order than the full layer's: bit-exact against the shards computed one by one on this
                    # GPU, within rounding against the unsharded layer.
                    step = n // world
                    want = torch.cat([hidet_b200.symmetric_quant_matmul(x, wq_full[:, r * step:(r + 1) * step].contiguous(),
                                                                        scale_full[r * step:(r + 1) * step].contiguous())
                                      for r in range(world)], dim=1)
                    full = hidet_b200.symmetric_quant_matmul(x, wq_full, scale_full)
                    assert (want.float() - full.float()).abs().max() <= 1e-3 * full.float().abs().max()
                    for call in range(3):  # repeated calls reuse (and alternate) the output buffers
                        got = layer(x)
                        torch.cuda.synchronize()
                        assert got.shape == want.shape
                        assert torch.equal(got, want), 'rank {} gather {} M {} call {}: {} differ'.format(
                            rank, gather, m, call, int((got != want).sum()))
                torch.cuda.synchronize()
                dist.barrier()
                layer.release()   # nothing peer-mapped may outlive the group
        assert hidet_b200.ffi.func('b200q_check_status')() == 0
        dist.barrier()
        if rank == 0:
            print('distributed gpu check ok on', world, 'GPUs')
    finally:
        dist.destroy_process_group()
    return 0


if __name__ == '__main__':
    sys.exit(main())
