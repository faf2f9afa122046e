"""The multi-GPU arm of bench.py: the 70B-shaped quantized linear, split column-parallel.

One process per GPU (torch.distributed, NCCL).  W int8 [8192, 28672] is split along N over the ranks,
activations fp16 [M, 8192] are replicated, every rank runs the single-GPU kernel on its shard and the
fp16 output slices are all-gathered, so every rank ends with the full [M, 28672] output.  M is swept
over {1, 16, 256, 2048}; a step is one pass over a rotation of distinct weight shards (larger than L2)
for every M.  Strong scaling: the layer is the same at every GPU count, `value` counts the whole
layer's algorithmic bytes, time is the maximum over ranks.
"""
from __future__ import annotations

import json
import os
import time

K_70B, N_70B = 8192, 28672
MS_70B = (1, 16, 256, 2048)


def algorithmic_bytes(m: int, k: int, n: int) -> int:
    return k * n + 2 * m * k + 2 * n + 2 * m * n


def run_sharded(args) -> int:
    import torch
    import torch.distributed as dist

    import hidet_b200
    from hidet_b200.distributed import ColumnParallelQuantLinear, column_range

    multicast = getattr(args, 'multicast', 'on') == 'on'
    if not multicast:
        # Plain peer mappings only: the outputs are written with ordinary stores.
        os.environ.setdefault('TORCH_SYMM_MEM_DISABLE_MULTICAST', '1')
    # (With multicast on, the outputs are also bound to an NVLink multicast object where the system has one, and large
    # M is delivered by single stores to it.  Memory bound to such an object must not be left behind by a rank that
    # ends early: every rank releases its layers before the process group goes, see the end of this function.)
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', str(args.gpus)))
    local_rank = int(os.environ.get('LOCAL_RANK', str(rank)))
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    if not dist.is_initialized():
        dist.init_process_group('nccl', device_id=device)

    from bench import ClockSampler, measured_peaks  # the launcher script

    peaks = measured_peaks()
    k, n = K_70B, N_70B
    global MS_70B
    if getattr(args, 'm_list', None):
        MS_70B = tuple(int(x) for x in args.m_list.split(','))
    if args.gather is None:
        args.gather = 'p2p'  # epilogue stores into the peer-mapped outputs; 'nccl' is the all-gather of the reference's op
    begin, end = column_range(n, rank, world)
    n_local = end - begin
    copies = max(2, -(-(2 * 128 * 1024 * 1024) // (k * n_local)))
    copies = min(copies, 16)

    # Every rank draws the same full-width weights from the same seeds and keeps its columns.
    layers = []
    for i in range(copies):
        gen = torch.Generator(device=device).manual_seed(100 + i)
        w = (torch.randn(k, n, generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.float16)
        layers.append(ColumnParallelQuantLinear.from_weight_shard(w[:, begin:end].contiguous(), gather=args.gather, multicast=multicast))
        if args.gather == 'p2p' and i > 0:
            layers[-1].share_outputs_with(layers[0])
        del w
    gen = torch.Generator(device=device).manual_seed(1)
    acts = {m: torch.randn(m, k, generator=gen, device=device, dtype=torch.float32).to(torch.float16) for m in MS_70B}

    def step(ms=MS_70B):
        out = None
        for m in ms:
            for layer in layers:
                out = layer(acts[m])
        return out

    def timed(fn, reps):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / reps

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()

    # Parity of the delivered result: the gathered [M, N] output of the first weight on this rank against the
    # same layer computed shard by shard on this GPU alone (every rank draws the full weight from the seed).
    gen = torch.Generator(device=device).manual_seed(100)
    w_full = (torch.randn(k, n, generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.float16)
    parity_ok = True
    for m in MS_70B:
        got = layers[0](acts[m]).clone()
        want = torch.empty(m, n, dtype=torch.float16, device=device)
        for r in range(world):
            b, e = column_range(n, r, world)
            wq_r, scale_r = hidet_b200.symmetric_quantize(w_full[:, b:e].contiguous(), 'int8', dims=0)
            want[:, b:e] = hidet_b200.symmetric_quant_matmul(acts[m], wq_r, scale_r)
        torch.cuda.synchronize()
        parity_ok = parity_ok and bool(torch.equal(got, want))
    del w_full
    flag = torch.tensor([1 if parity_ok else 0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    parity_ok = bool(flag.item())
    assert parity_ok, 'the gathered output differs from the shard-by-shard result'

    # Replay each sweep as one CUDA graph when the whole step can be captured (kernel launches and the
    # cross-rank barrier are ordinary stream work); otherwise launch eagerly.
    side = torch.cuda.Stream(device)
    graphs = {}
    timing = 'eager launches'
    if not args.eager:
        try:
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for key in (MS_70B,) + tuple((m,) for m in MS_70B):
                    step(key)  # buffers and workspaces for this stream exist before capture
                    side.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        step(key)
                    graphs[key] = g
                    del g
            timing = 'one CUDA graph per sweep'
        except Exception as e:  # capture is an optimisation of the measurement, not part of the product
            graphs = {}
            timing = 'eager launches (graph capture unavailable: {})'.format(str(e).splitlines()[0][:120])
            torch.cuda.synchronize()
    flags = torch.tensor([1 if graphs else 0], device=device)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if int(flags.item()) == 0:
        graphs = {}

    def run(key=MS_70B):
        if graphs:
            graphs[key].replay()
        else:
            step(key)

    if graphs:
        torch.cuda.set_stream(side)
    with ClockSampler(local_rank) as clocks:
        time.sleep(0.15)
        ms_per_step = timed(run, args.steps)
        if ms_per_step * args.steps < 400.0:
            for _ in range(int(400.0 / max(ms_per_step, 1e-3)) + 1):
                run()
            torch.cuda.synchronize()
    bytes_per_step = sum(algorithmic_bytes(m, k, n) * copies for m in MS_70B)
    flops_per_step = sum(2.0 * m * k * n * copies for m in MS_70B)
    value = bytes_per_step / (ms_per_step * 1e-3) / 1e9

    shapes = []
    for m in MS_70B:
        ms_m = timed(lambda: run((m,)), 5)
        us = ms_m * 1e3 / copies
        shapes.append({'M': m, 'K': k, 'N': n, 'us_per_layer': round(us, 2), 'GBps': round(algorithmic_bytes(m, k, n) / us / 1e3, 1),
                       'TFLOPS': round(2.0 * m * k * n / us / 1e6, 2)})
        # the same without the gather: what the delivery costs
        c_local = torch.empty(m, n_local, dtype=torch.float16, device=device)

        def local_only():
            for layer in layers:
                layer.local(acts[m], out=c_local)

        local_only()
        g_local = None
        if graphs:
            torch.cuda.current_stream().synchronize()
            g_local = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_local, stream=torch.cuda.current_stream()):
                local_only()
        us_local = timed((lambda: g_local.replay()) if g_local is not None else local_only, 5) * 1e3 / copies
        shapes[-1]['us_local_kernel'] = round(us_local, 2)
        del g_local

    # The same layer, unsharded, on this GPU alone (every rank does it at once, without communication; rank 0's
    # time is reported): what the sharded layer is to be compared with.
    one_gpu = []
    full_layers = []
    for i in range(2):
        gen = torch.Generator(device=device).manual_seed(100 + i)
        w = (torch.randn(k, n, generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.float16)
        full_layers.append(hidet_b200.symmetric_quantize(w, 'int8', dims=0))
        del w
    for m in MS_70B:
        out_full = torch.empty(m, n, dtype=torch.float16, device=device)

        def full_pass():
            for wq_full, scale_full in full_layers:
                hidet_b200.symmetric_quant_matmul(acts[m], wq_full, scale_full, out=out_full)

        full_pass()
        g_full = None
        if graphs:
            torch.cuda.current_stream().synchronize()
            g_full = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_full, stream=torch.cuda.current_stream()):
                for _ in range(4):
                    full_pass()
        us_full = timed((lambda: g_full.replay()) if g_full is not None else (lambda: [full_pass() for _ in range(4)]), 5) * 1e3 / (4 * len(full_layers))
        one_gpu.append(round(us_full, 2))
        del g_full
    for entry, us_full in zip(shapes, one_gpu):
        entry['us_per_layer_one_gpu'] = us_full
        entry['speedup_vs_one_gpu'] = round(us_full / entry['us_per_layer'], 2)
    del full_layers

    # end to end: activations from pinned host memory in, gathered output back to the host, every step
    pinned_in = {m: acts[m].cpu().pin_memory() for m in MS_70B}
    pinned_out = {m: torch.empty(m, n, dtype=torch.float16).pin_memory() for m in MS_70B}

    def e2e_step():
        for m in MS_70B:
            acts[m].copy_(pinned_in[m], non_blocking=True)
            out = None
            for layer in layers:
                out = layer(acts[m])
            pinned_out[m].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_step()
    e2e_ms = timed(e2e_step, max(args.steps // 2, 3))
    e2e_value = bytes_per_step / (e2e_ms * 1e-3) / 1e9
    assert hidet_b200.ffi.func('b200q_check_status')() == 0

    if rank == 0:
        uses_multicast = args.gather == 'p2p' and any(po.multicast_ptrs and po.multicast_ptrs[0] for layer in layers for po in layer._peer_outputs.values())
        large_m_delivery = ('one multimem.st per 16 bytes to the NVLink multicast mapping of the outputs'
                            if uses_multicast and multicast and world >= ColumnParallelQuantLinear.MULTICAST_MIN_WORLD
                            else 'peer stores to every rank' if args.gather == 'p2p' else 'NCCL all-gather')
        line = {
            'metric': 'quant-linear HBM GB/s (70B-shaped layer, column-parallel)', 'value': value, 'unit': 'GB/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': ms_per_step, 'higher_is_better': True,
            'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f16', 'accumulate': 'f32', 'weight_dtype': 'i8', 'data': 'synthetic',
            'config': {'workload': 'sharded-70b-layer', 'K': k, 'N': n, 'M': list(MS_70B), 'parallelism': 'tp{} (columns), outputs by {}'.format(world, 'peer stores from the kernels\' epilogues + one cross-rank barrier' if args.gather == 'p2p' else 'NCCL all-gather'),
                       'large_m_delivery': large_m_delivery,
                       'weights_in_rotation': copies, 'l2': 'inputs larger than L2: {} distinct weight shards of {} MB per rank'.format(copies, k * n_local // 1000000),
                       'timing': timing + ', CUDA events, barrier on both sides, max over ranks'},
            'tflops': flops_per_step / (ms_per_step * 1e-3) / 1e12,
            'gpu_launches': len(MS_70B) * copies * args.steps,
            'parity_checked': parity_ok,
            'clocks': clocks.summary(),
            'roofline': {'bound': 'hbm for M <= 16, tensor for M >= 256', 'achieved': value, 'peak': peaks['hbm_gbs'] * world, 'unit': 'GB/s',
                         'frac': value / (peaks['hbm_gbs'] * world), 'traffic': None, 'peak_source': peaks['source'] + ' (burst copy) x n_gpus',
                         'kernel': 'qlinear_decode_kn_kernel / qlinear_prefill_kn_kernel' + (' + ncclAllGather' if args.gather == 'nccl' else ' (peer stores)')},
            'shapes': shapes,
            'e2e': {'value': e2e_value, 'unit': 'GB/s', 'h2d_bytes_per_step': sum(t.numel() * 2 for t in pinned_in.values()),
                    'd2h_bytes_per_step': sum(t.numel() * 2 for t in pinned_out.values()), 'ms_per_step': e2e_ms},
        }
        line['speedup_vs_one_gpu'] = round(sum(one_gpu) / sum(e['us_per_layer'] for e in shapes), 2)
        print(json.dumps(line), flush=True)
    # Captured collectives keep the communicator alive, and peer-mapped outputs must not outlive a rank:
    # release the graphs and everything that maps another GPU's memory before the process group goes.
    import gc

    graphs.clear()
    torch.cuda.synchronize()
    dist.barrier()
    for layer in layers:
        layer.release()
    layers.clear()
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    _exit_if_teardown_stalls(10.0)
    dist.destroy_process_group()
    return 0


def _exit_if_teardown_stalls(seconds: float) -> None:
    """The result is printed and every rank has passed the last barrier; a communicator teardown that does not
    finish in `seconds` must not keep the GPUs."""
    import sys
    import threading

    def watchdog():
        time.sleep(seconds)
        sys.stdout.flush()
        sys.stderr.write('bench: process group teardown still running after {:.0f} s, exiting\n'.format(seconds))
        sys.stderr.flush()
        os._exit(0)

    threading.Thread(target=watchdog, daemon=True).start()
