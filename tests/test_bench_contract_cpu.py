"""The reference arm of bench.py runs on the host cores alone: its JSON line is checked here, without a GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(extra_env=None, gpus=1):
    env = dict(os.environ)
    for key in ('RANK', 'LOCAL_RANK', 'WORLD_SIZE'):
        env.pop(key, None)
    env.update(extra_env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, 'bench.py'), '--impl', 'reference', '--gpus', str(gpus), '--steps', '1', '--warmup', '1'],
                          cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)


def test_reference_arm_prints_one_line_with_the_contract_keys():
    done = _run()
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [ln for ln in done.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line['impl'] == 'reference'
    for key in ('metric', 'value', 'unit', 'n_gpus', 'steps', 'warmup', 'ms_per_step', 'higher_is_better', 'scaling', 'vs_baseline',
                'dtype', 'data', 'config', 'cpu_baseline', 'e2e'):
        assert key in line, key
    assert line['unit'] == 'GB/s' and line['higher_is_better'] is True and line['vs_baseline'] is None
    assert line['value'] > 0 and line['ms_per_step'] > 0
    assert line['config']['workload'] == 'decode-llama7b'
    base = line['cpu_baseline']
    assert base['kind'] in ('port', 'reference') and base['cores'] >= 1 and base['sample'] and base['value'] == line['value']
    e2e = line['e2e']
    assert e2e['value'] == line['value'] and e2e['unit'] == line['unit']
    assert e2e['h2d_bytes_per_step'] == 0 and e2e['d2h_bytes_per_step'] == 0


def test_reference_arm_runs_on_rank_zero_only():
    done = _run({'RANK': '1', 'LOCAL_RANK': '1', 'WORLD_SIZE': '2'}, gpus=2)
    assert done.returncode == 0, done.stderr[-2000:]
    assert done.stdout.strip() == ''
