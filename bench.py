"""Benchmark of the weight-only int8 quantized linear path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One GPU (the default): the decode configuration -- activations fp16 [M, 4096] for M in {1, 4, 16}
against int8 weights [4096, N], N in {4096, 11008}, per-column fp16 scales, fp32 accumulation, fp16
output.  A step is one pass over a stack of distinct weight matrices (16 of the 4096-wide, 6 of the
11008-wide, together larger than twice the L2 cache, so every weight is streamed from HBM) for each M:
66 kernel launches.  `value` is algorithmic bytes per second (each tensor counted once:
K*N + 2*M*K + 2*N + 2*M*N per launch).

More than one GPU (launched through torch.distributed.run, one rank per GPU): the 70B-shaped layer
(K = 8192, N = 28672, M swept over {1, 16, 256, 2048}) split column-parallel over the ranks with an
all-gather of the fp16 output slices; strong scaling, time is the maximum over ranks.

--impl reference times the reference's CPU arithmetic for the same configuration (the CPU oracle built
with the reference's own compiler flags) on this host's cores.

Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

K_DECODE = 4096
DECODE_NS = (4096, 11008)
DECODE_MS = (1, 4, 16)
STACK = {4096: 16, 11008: 6}  # distinct weight matrices per width: 268 MB + 270 MB of int8
TRAFFIC_FILE = os.path.join(ROOT, 'profiles', 'qlinear_decode_dram_traffic.json')
DECODE_SOURCE = os.path.join(ROOT, 'hidet_b200', 'csrc', 'qlinear_decode.cu')


def source_digest(path: str = DECODE_SOURCE) -> str:
    import hashlib

    with open(path, 'rb') as f:
        return hashlib.sha256(f.read()).hexdigest()[:16]


def record_traffic(csv_paths) -> int:
    """Reads ncu CSV logs of `bench.py --case M,K,N --eager` captures (metrics dram__bytes_read.sum and
    dram__bytes_write.sum of the small-M kernel; the case is taken from the file name, decode_M,K,N.csv) and
    writes profiles/qlinear_decode_dram_traffic.json: DRAM bytes per launch by shape, with the digest of the
    kernel source they were measured on."""
    import csv
    import re

    per_case = {}
    for path in csv_paths:
        m = re.search(r'(\d+),(\d+),(\d+)', os.path.basename(path))
        if not m:
            raise SystemExit('cannot tell the case from the file name {}'.format(path))
        launches = {}
        with open(path, newline='') as f:
            for row in csv.reader(f):
                if len(row) >= 15 and row[12] in ('dram__bytes_read.sum', 'dram__bytes_write.sum') and 'qlinear_decode' in row[4]:
                    scale = {'byte': 1, 'Kbyte': 1e3, 'Mbyte': 1e6, 'Gbyte': 1e9}[row[13]]
                    launches.setdefault(row[0], 0.0)
                    launches[row[0]] += float(row[14].replace(',', '')) * scale
        if not launches:
            raise SystemExit('no DRAM counters of the small-M kernel in {}'.format(path))
        per_case['{},{},{}'.format(*m.groups())] = sum(launches.values()) / len(launches)
    with open(TRAFFIC_FILE, 'w') as f:
        json.dump({'kernel_source_sha256_16': source_digest(), 'unit': 'bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum)',
                   'cases': per_case}, f, indent=1)
        f.write('\n')
    print('wrote', TRAFFIC_FILE)
    return 0


def ncu_traffic_per_launch():
    """Average DRAM traffic per launch over the launch mix of one step, from the recorded ncu capture of the kernel
    as it is now: None when there is no record, when it was taken on another version of the kernel source, or when
    a shape is missing (M = 4 was not captured and is taken on the line between M = 1 and M = 16)."""
    try:
        with open(TRAFFIC_FILE) as f:
            rec = json.load(f)
        if rec.get('kernel_source_sha256_16') != source_digest():
            return None
        total, launches = 0.0, 0
        for n, count in STACK.items():
            lo, hi = rec['cases']['1,{},{}'.format(K_DECODE, n)], rec['cases']['16,{},{}'.format(K_DECODE, n)]
            for m in DECODE_MS:
                total += count * rec['cases'].get('{},{},{}'.format(m, K_DECODE, n), lo + (hi - lo) * (m - 1) / 15.0)
                launches += count
        return total / launches
    except (OSError, KeyError, ValueError):
        return None


K_70B, N_70B = 8192, 28672
MS_70B = (1, 16, 256, 2048)


def algorithmic_bytes(m: int, k: int, n: int) -> int:
    return k * n + 2 * m * k + 2 * n + 2 * m * n


def measured_peaks() -> dict:
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {'hbm_gbs': float(d['hbm_gbs']), 'bf16_tflops': float(d['bf16_tflops']),
                'bf16_tflops_sustained': float(d.get('bf16_tflops_sustained', d['bf16_tflops'])), 'source': 'measured'}
    return {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0, 'source': 'fallback'}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    QUERY = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self.thread = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', '-i', str(self.index), '--query-gpu=' + self.QUERY, '--format=csv,noheader,nounits', '-lms', '100'],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self) -> dict:
        sm, sm_max, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for line in self.lines:
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                sm_max.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        if not sm:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        return {'sm_mhz': statistics.median(sm), 'sm_max_mhz': max(sm_max), 'reasons': sorted(reasons), 'samples': len(sm)}


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's x86 arithmetic (the oracle port) on this host's cores
# ---------------------------------------------------------------------------------------------
def build_cpu_port():
    """The oracle compiled with the reference's CPU flags (-O3 -mavx2 -ffast-math -march=native -fopenmp).
    -march=native must be resolved on the machine that runs the code, so this is built here, now."""
    import oracle

    tmp = tempfile.mkdtemp(prefix='b200q_cpu_')
    try:
        path = oracle.build(os.path.join(tmp, 'libquant_oracle_ref_flags.so'), oracle.REFERENCE_FLAGS, force=True)
        kind_note = 'reference build flags'
    except Exception:
        path = oracle.build()
        kind_note = 'portable build'
    return oracle, oracle.load(path), kind_note


def cpu_decode_pass(oracle, lib, rng_seed: int = 0):
    """One weight per (M, N) of the decode configuration through the reference's x86 loop
    (float32 activations, int8 weights dequantized inside the loop).  Returns (bytes, seconds)."""
    import numpy as np

    rng = np.random.default_rng(rng_seed)
    total_bytes, total_s = 0, 0.0
    for n in DECODE_NS:
        wq = rng.integers(-127, 128, size=(K_DECODE, n), dtype=np.int8)
        scale = np.full((n,), 5e-4, dtype=np.float32)
        for m in DECODE_MS:
            a = rng.standard_normal((m, K_DECODE), dtype=np.float32)
            t0 = time.perf_counter()
            oracle.symmetric_quant_matmul(a, wq, scale, lib=lib)
            total_s += time.perf_counter() - t0
            total_bytes += algorithmic_bytes(m, K_DECODE, n)
    return total_bytes, total_s


def cpu_baseline_block(passes: int = 3):
    oracle, lib, note = build_cpu_port()
    cpu_decode_pass(oracle, lib)  # warm-up: page in, spin up the OpenMP team
    best = None
    for _ in range(passes):
        b, s = cpu_decode_pass(oracle, lib)
        gbs = b / s / 1e9
        best = gbs if best is None else max(best, gbs)
    return {
        'value': best, 'unit': 'GB/s', 'cores': oracle.num_threads(lib), 'kind': 'port',
        'sample': 'one weight per (M, N) of the step (6 of its 66 launches), float32 activations, the reference x86 loop, '
                  'best of {} passes, {}'.format(passes, note),
    }


def run_reference_arm(args) -> int:
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return 0
    oracle, lib, note = build_cpu_port()
    for _ in range(max(args.warmup, 1)):
        cpu_decode_pass(oracle, lib)
    t_total, b_total = 0.0, 0
    for _ in range(args.steps):
        b, s = cpu_decode_pass(oracle, lib)
        t_total += s
        b_total += b
    value = b_total / t_total / 1e9
    cores = oracle.num_threads(lib)
    sample = ('each step = one weight per (M, N) of the decode configuration (6 of the 66 launches of a full step), float32 '
              'activations, the reference x86 loop, ' + note)
    line = {
        'impl': 'reference', 'metric': 'quant-linear HBM GB/s (decode)', 'value': value, 'unit': 'GB/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': 1e3 * t_total / args.steps, 'higher_is_better': True,
        'scaling': 'weak' if args.gpus == 1 else 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': 'decode-llama7b', 'K': K_DECODE, 'N': list(DECODE_NS), 'M': list(DECODE_MS)},
        'cpu_baseline': {'value': value, 'unit': 'GB/s', 'cores': cores, 'kind': 'port', 'sample': sample},
        'e2e': {'value': value, 'unit': 'GB/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def make_quantized_stack(torch, hidet_b200, device, k: int, n: int, count: int, seed: int):
    """`count` distinct int8 [k, n] weights with their fp16 scales, quantized on the device from
    W ~ N(0, 0.02^2) fp16."""
    gen = torch.Generator(device=device).manual_seed(seed)
    out = []
    for _ in range(count):
        w = (torch.randn(k, n, generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.float16)
        wq, scale = hidet_b200.symmetric_quantize(w, 'int8', dims=0)
        out.append((wq, scale))
        del w
    return out


def time_graph(torch, stream, fn, launches_per_call: int, min_calls: int = 5, min_ms: float = 20.0):
    """Average device time of one launch of `fn`'s launches: `fn` is captured into a CUDA graph on
    `stream` and replayed between two events until at least `min_ms` have passed."""
    fn()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        fn()
    for _ in range(3):
        graph.replay()
    calls = min_calls
    while True:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        e0.record(stream)
        for _ in range(calls):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
        ms = e0.elapsed_time(e1)
        if ms >= min_ms or calls >= 4096:
            return ms * 1e3 / (calls * launches_per_call)
        calls *= 4


def extra_sections(torch, hidet_b200, device, stream, peaks):
    """Prefill shapes and the quantize kernel, timed the same way; reported beside the headline."""
    out = {}
    prefill = []
    for m, k, n in ((2048, 4096, 11008), (2048, 11008, 4096)):
        stack = make_quantized_stack(torch, hidet_b200, device, k, n, 4, seed=k)
        gen = torch.Generator(device=device).manual_seed(2)
        a = torch.randn(m, k, generator=gen, device=device, dtype=torch.float32).to(torch.float16)
        outs = [torch.empty(m, n, dtype=torch.float16, device=device) for _ in stack]

        def fn():
            for (wq, scale), c in zip(stack, outs):
                hidet_b200.symmetric_quant_matmul(a, wq, scale, out=c)

        us = time_graph(torch, stream, fn, len(stack))
        flops = 2.0 * m * k * n
        prefill.append({'M': m, 'K': k, 'N': n, 'us_per_launch': round(us, 2), 'TFLOPS': round(flops / us / 1e6, 1),
                        'frac_of_bf16_burst_peak': round(flops / us / 1e6 / peaks['bf16_tflops'], 4),
                        'frac_of_bf16_sustained_peak': round(flops / us / 1e6 / peaks['bf16_tflops_sustained'], 4)})
        del stack, outs
    out['prefill'] = prefill
    k, n = 4096, 4096
    gen = torch.Generator(device=device).manual_seed(3)
    ws = [(torch.randn(k, n, generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.float16) for _ in range(8)]  # 268 MB > L2

    def qfn():
        for w in ws:
            hidet_b200.symmetric_quantize(w, 'int8', dims=0)

    us = time_graph(torch, stream, qfn, len(ws))  # outputs come from the graph's private pool
    qbytes = 3 * k * n + 2 * n
    out['quantize'] = {'K': k, 'N': n, 'dtype': 'f16->i8, dims=0', 'us_per_launch': round(us, 2), 'GBps': round(qbytes / us / 1e3, 1),
                       'frac_of_hbm_peak': round(qbytes / us / 1e3 / peaks['hbm_gbs'], 4)}
    del ws
    # quantize and dequantize over the projection shapes, both reduced dimensions
    family = []
    for k, n in ((4096, 4096), (4096, 11008), (11008, 4096)):
        count = 8 if k * n < 3e7 else 4   # > L2 in rotation either way
        ws = [(torch.randn(k, n, generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.float16) for _ in range(count)]
        for dims in (0, -1):
            def qfn():
                for w in ws:
                    hidet_b200.symmetric_quantize(w, 'int8', dims=dims)

            q_us = time_graph(torch, stream, qfn, len(ws))
            qs = [hidet_b200.symmetric_quantize(w, 'int8', dims=dims) for w in ws]

            def dfn():
                for wq, sc in qs:
                    hidet_b200.symmetric_dequantize(wq, sc, dims=dims)

            d_us = time_graph(torch, stream, dfn, len(qs))
            del qs
            nbytes = 3 * k * n
            family.append({'rows': k, 'cols': n, 'dims': dims,
                           'quantize_us': round(q_us, 2), 'quantize_frac_of_hbm_peak': round(nbytes / q_us / 1e3 / peaks['hbm_gbs'], 4),
                           'dequantize_us': round(d_us, 2), 'dequantize_frac_of_hbm_peak': round(nbytes / d_us / 1e3 / peaks['hbm_gbs'], 4)})
        del ws
    out['quantize_family'] = family
    # The 70B-shaped layer of the multi-GPU runs, unsharded on this one GPU: the base of their speed-up.
    stack = make_quantized_stack(torch, hidet_b200, device, K_70B, N_70B, 2, seed=70)
    one_gpu = []
    for m in MS_70B:
        gen = torch.Generator(device=device).manual_seed(4)
        a = torch.randn(m, K_70B, generator=gen, device=device, dtype=torch.float32).to(torch.float16)
        c = torch.empty(m, N_70B, dtype=torch.float16, device=device)

        def fn70():
            for wq, scale in stack:
                hidet_b200.symmetric_quant_matmul(a, wq, scale, out=c)

        us = time_graph(torch, stream, fn70, len(stack))
        one_gpu.append({'M': m, 'K': K_70B, 'N': N_70B, 'us_per_layer_one_gpu': round(us, 2),
                        'GBps': round(algorithmic_bytes(m, K_70B, N_70B) / us / 1e3, 1), 'TFLOPS': round(2.0 * m * K_70B * N_70B / us / 1e6, 1)})
    out['sharded_70b_one_gpu'] = one_gpu
    del stack
    # 4-bit weights with group scales and zero points (the shapes and group size of the reference's own test program,
    # tests/cute_kernel/test_quant_linear.py:53-61): bytes = the packed codes + scales + zero points + activations + output.
    from hidet_b200.quant import cast_f16_to_u4, w4a16_linear

    w4 = []
    for m, n, k in ((1, 4096, 4096), (1, 12288, 4096), (1, 4096, 12288)):
        gsize = 128
        gen = torch.Generator(device=device).manual_seed(5)
        count = max(12, -(-160_000_000 // (k * n // 2)))  # 160 to 300 MB of codes in rotation: larger than L2
        codes = [cast_f16_to_u4(torch.randint(0, 16, (k, n), device=device, generator=gen).to(torch.float16)) for _ in range(count)]
        scale = (torch.rand(k // gsize, n, device=device, generator=gen) * 0.01).to(torch.float16)
        zeros = (torch.rand(k // gsize, n, device=device, generator=gen) * 15).to(torch.float16)
        a = torch.randn(m, k, generator=gen, device=device, dtype=torch.float32).to(torch.float16)
        linear = w4a16_linear('bench', k, n, gsize, with_zp=True)

        def fn4():
            for q in codes:
                linear(a, q, scale, zeros)

        us = time_graph(torch, stream, fn4, count)
        nbytes = k * n // 2 + 2 * 2 * (k // gsize) * n + 2 * m * k + 2 * m * n
        w4.append({'M': m, 'K': k, 'N': n, 'group_size': gsize, 'us_per_launch': round(us, 2), 'GBps': round(nbytes / us / 1e3, 1),
                   'frac_of_hbm_peak': round(nbytes / us / 1e3 / peaks['hbm_gbs'], 4)})
        del codes
    out['w4a16'] = w4
    return out


def run_single_gpu(args) -> int:
    import torch

    import hidet_b200

    torch.cuda.set_device(0)
    device = torch.device('cuda', 0)
    peaks = measured_peaks()

    stacks = {n: make_quantized_stack(torch, hidet_b200, device, K_DECODE, n, STACK[n], seed=n) for n in DECODE_NS}
    gen = torch.Generator(device=device).manual_seed(1)
    acts = {m: torch.randn(m, K_DECODE, generator=gen, device=device, dtype=torch.float32).to(torch.float16) for m in DECODE_MS}
    outs = {(m, n): [torch.empty(m, n, dtype=torch.float16, device=device) for _ in range(STACK[n])]
            for m in DECODE_MS for n in DECODE_NS}
    launches_per_step = len(DECODE_MS) * sum(STACK.values())
    bytes_per_step = sum(algorithmic_bytes(m, K_DECODE, n) * STACK[n] for m in DECODE_MS for n in DECODE_NS)
    flops_per_step = sum(2 * m * K_DECODE * n * STACK[n] for m in DECODE_MS for n in DECODE_NS)

    def step(ms=DECODE_MS, ns=DECODE_NS):
        for m in ms:
            for n in ns:
                for (wq, scale), c in zip(stacks[n], outs[(m, n)]):
                    hidet_b200.symmetric_quant_matmul(acts[m], wq, scale, out=c)

    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(max(args.warmup, 3)):
            step()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        side.synchronize()

        # ---- timed region: exactly `steps` replays between two events on the launching stream ----
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(0) as clocks:
            time.sleep(0.15)
            side.synchronize()
            start.record(side)
            for _ in range(args.steps):
                graph.replay()
            stop.record(side)
            side.synchronize()
            elapsed_ms = start.elapsed_time(stop)
            if elapsed_ms < 400.0:  # keep the GPU busy long enough for a few clock samples
                reps = int(400.0 / max(elapsed_ms / args.steps, 1e-3)) + 1
                for _ in range(reps):
                    graph.replay()
                side.synchronize()
        ms_per_step = elapsed_ms / args.steps
        value = bytes_per_step / (ms_per_step * 1e-3) / 1e9

        # ---- per-shape breakdown (same stack, one graph per shape) ----
        shapes = []
        for m in DECODE_MS:
            for n in DECODE_NS:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    step((m,), (n,))
                for _ in range(3):
                    g.replay()
                reps = 20
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                side.synchronize()
                e0.record(side)
                for _ in range(reps):
                    g.replay()
                e1.record(side)
                side.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / (reps * STACK[n])
                b = algorithmic_bytes(m, K_DECODE, n)
                shapes.append({'M': m, 'K': K_DECODE, 'N': n, 'us_per_launch': round(us, 3), 'GBps': round(b / us / 1e3, 1),
                               'TFLOPS': round(2 * m * K_DECODE * n / us / 1e6, 3),
                               'frac_of_hbm_peak': round(b / us / 1e3 / peaks['hbm_gbs'], 4)})

    # ---- end to end through the public API: host activations in, host result out, every step ----
    pinned_in = {m: acts[m].cpu().pin_memory() for m in DECODE_MS}
    pinned_out = {m: torch.empty(m, DECODE_NS[-1], dtype=torch.float16).pin_memory() for m in DECODE_MS}
    h2d = sum(t.numel() * 2 for t in pinned_in.values())
    d2h = sum(t.numel() * 2 for t in pinned_out.values())

    # One hidet_b200.CudaGraph per M: the public replay API (the counterpart of the reference's CUDA-graph mode).
    def make_graph(m):
        def f_run(inputs):
            last = None
            for n in DECODE_NS:
                for (wq, scale), c in zip(stacks[n], outs[(m, n)]):
                    last = hidet_b200.symmetric_quant_matmul(inputs[0], wq, scale, out=c)
            return [last]

        return hidet_b200.CudaGraph(lambda: [acts[m]], f_run, ref_objs=[stacks])

    e2e_graphs = {m: make_graph(m) for m in DECODE_MS}

    def e2e_step():
        for m in DECODE_MS:
            (last,) = e2e_graphs[m].run_async([pinned_in[m]])      # host -> device copy of the activations, then replay
            pinned_out[m].copy_(last, non_blocking=True)           # device -> host read of the result
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    e2e_steps = max(args.steps, 5)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    e2e_value = bytes_per_step / (e2e_ms * 1e-3) / 1e9
    del e2e_graphs

    extras = {}
    if not args.no_extras:
        del stacks, outs
        with torch.cuda.stream(side):
            extras = extra_sections(torch, hidet_b200, device, side, peaks)

    if not args.no_extras and not args.no_config4:
        import bench_decoder

        torch.cuda.empty_cache()
        extras['config4'] = bench_decoder.run_config(bench_decoder.LLAMA_7B)
    status = hidet_b200.ffi.func('b200q_check_status')()
    assert status == 0

    line = {
        'metric': 'quant-linear HBM GB/s (decode)', 'value': value, 'unit': 'GB/s', 'n_gpus': 1, 'steps': args.steps,
        'warmup': max(args.warmup, 3), 'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'weak',
        'vs_baseline': None, 'dtype': 'f16', 'accumulate': 'f32', 'weight_dtype': 'i8', 'data': 'synthetic',
        'config': {'workload': 'decode-llama7b', 'K': K_DECODE, 'N': list(DECODE_NS), 'M': list(DECODE_MS),
                   'weights_per_step': dict((str(k), v) for k, v in STACK.items()), 'launches_per_step': launches_per_step,
                   'l2': 'inputs larger than L2: 538 MB of distinct int8 weights per pass', 'timing': 'one CUDA graph per step, CUDA events on the launching stream'},
        'tflops': flops_per_step / (ms_per_step * 1e-3) / 1e12,
        'gpu_launches': launches_per_step * args.steps,
        'clocks': clocks.summary(),
        'roofline': {'bound': 'hbm', 'achieved': value, 'peak': peaks['hbm_gbs'], 'unit': 'GB/s', 'frac': value / peaks['hbm_gbs'],
                     'traffic': ncu_traffic_per_launch(),
                     'traffic_unit': 'DRAM bytes per launch from the recorded ncu capture of this kernel source, averaged over the step\'s launch mix; '
                                     'null: no capture of the kernel as it is now (algorithmic_bytes_per_launch is the algorithmic figure)',
                     'algorithmic_bytes_per_launch': bytes_per_step / launches_per_step,
                     'peak_source': peaks['source'] + ' (burst copy)', 'kernel': 'qlinear_decode_kn_kernel'},
        'shapes': shapes,
        'e2e': {'value': e2e_value, 'unit': 'GB/s', 'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h, 'ms_per_step': e2e_ms,
                'note': 'hidet_b200.CudaGraph.run_async per M (pinned host activations copied in, 22 quantized linears replayed), result copied back to pinned host memory, one synchronisation per step'},
    }
    line.update(extras)
    if not args.no_cpu_baseline:
        line['cpu_baseline'] = cpu_baseline_block()
    print(json.dumps(line))
    return 0


def run_case(args) -> int:
    """One shape, a rotation of distinct weights larger than L2, eager launches: the small case that
    profiler captures and kernel tuning use.  Prints the average launch time from CUDA events."""
    import torch

    import hidet_b200

    m, k, n = (int(x) for x in args.case.split(','))
    torch.cuda.set_device(0)
    device = torch.device('cuda', 0)
    peaks = measured_peaks()
    count = max(2, -(-(2 * 128 * 1024 * 1024) // (k * n)))
    count = min(count, 64)
    layout = args.layout
    stack = make_quantized_stack(torch, hidet_b200, device, k, n, count, seed=7)
    if layout == 'NK':
        stack = [(wq.t().contiguous(), scale) for wq, scale in stack]
    gen = torch.Generator(device=device).manual_seed(1)
    a = torch.randn(m, k, generator=gen, device=device, dtype=torch.float32).to(torch.float16)
    outs = [torch.empty(m, n, dtype=torch.float16, device=device) for _ in range(count)]

    def one_pass():
        for (wq, scale), c in zip(stack, outs):
            hidet_b200.symmetric_quant_matmul(a, wq, scale, weight_layout=layout, out=c)

    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        one_pass()
        side.synchronize()
        if args.eager:
            runner = one_pass
        else:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                one_pass()
            runner = graph.replay
        passes = max(1, args.launches // count)
        for _ in range(min(3, passes)):
            runner()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        side.synchronize()
        e0.record(side)
        for _ in range(passes):
            runner()
        e1.record(side)
        side.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (passes * count)
    b = algorithmic_bytes(m, k, n)
    flops = 2.0 * m * k * n
    assert hidet_b200.ffi.func('b200q_check_status')() == 0
    print(json.dumps({'case': {'M': m, 'K': k, 'N': n, 'layout': layout}, 'weights_in_rotation': count, 'launches': passes * count,
                      'us_per_launch': us, 'GBps': b / us / 1e3, 'TFLOPS': flops / us / 1e6,
                      'frac_of_hbm_peak': b / us / 1e3 / peaks['hbm_gbs'], 'frac_of_bf16_burst_peak': flops / us / 1e6 / peaks['bf16_tflops']}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', choices=['ours', 'reference'], default='ours')
    ap.add_argument('--no-cpu-baseline', action='store_true', help='skip the CPU leg (for profiling runs)')
    ap.add_argument('--no-extras', action='store_true', help='skip the prefill and quantize sections (for profiling runs)')
    ap.add_argument('--gather', choices=['nccl', 'p2p'], default=None,
                    help='multi-GPU: how output slices reach every rank (default: p2p up to four GPUs, nccl on eight)')
    ap.add_argument('--multicast', choices=['on', 'off'], default='on',
                    help='multi-GPU, --gather p2p: deliver large M through the NVLink multicast mapping of the outputs where there is one')
    ap.add_argument('--m-list', default=None, help='multi-GPU: comma-separated activation row counts to sweep instead of 1,16,256,2048')
    ap.add_argument('--record-traffic', nargs='+', default=None, metavar='CSV',
                    help='no benchmark: read ncu CSV logs (decode_M,K,N.csv) and write profiles/qlinear_decode_dram_traffic.json')
    ap.add_argument('--config4', action='store_true', help='run only the Llama-2-7B-shaped decoder (512-token prompt, 128 greedy steps) and print its block')
    ap.add_argument('--no-config4', action='store_true', help='leave the decoder block out of the default line')
    ap.add_argument('--case', default=None, help='M,K,N: time one shape only (small case for profiling and tuning)')
    ap.add_argument('--layout', choices=['KN', 'NK'], default='KN', help='weight layout for --case')
    ap.add_argument('--launches', type=int, default=200, help='launches to time for --case')
    ap.add_argument('--eager', action='store_true', help='launch one by one instead of replaying a CUDA graph (--case and multi-GPU)')
    args = ap.parse_args(argv)
    if args.record_traffic:
        return record_traffic(args.record_traffic)
    if args.case:
        return run_case(args)
    if args.config4:
        import bench_decoder

        print(json.dumps({'config4': bench_decoder.run_config(bench_decoder.LLAMA_7B)}))
        return 0
    if args.impl == 'reference':
        return run_reference_arm(args)
    if args.gpus > 1 or int(os.environ.get('WORLD_SIZE', '1')) > 1:
        from bench_sharded import run_sharded

        return run_sharded(args)
    return run_single_gpu(args)


if __name__ == '__main__':
    sys.exit(main())
