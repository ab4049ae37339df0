"""The benchmark's command-line contract, as far as it can be checked without a GPU: the reference arm prints
exactly one JSON line with the agreed keys (it times the reference's serial CPU kernel on a bounded sample), and
the arm that measures this library refuses to run without a CUDA device instead of falling back to the CPU."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=600):
  return subprocess.run([sys.executable, os.path.join(ROOT, 'bench.py'), *args], cwd=ROOT, capture_output=True,
                        text=True, timeout=timeout)


def test_reference_arm_prints_one_json_line_with_the_agreed_keys():
  r = _run('--impl', 'reference', '--steps', '1', '--warmup', '0')
  assert r.returncode == 0, r.stderr[-2000:]
  lines = [l for l in r.stdout.splitlines() if l.startswith('{')]
  assert len(lines) == 1
  d = json.loads(lines[0])
  assert d['impl'] == 'reference' and d['metric'] == 'synaptic_ops_per_sec' and d['unit'] == 'SyOp/s'
  assert d['value'] > 0 and d['ms_per_step'] > 0 and d['higher_is_better'] is True
  assert d['n_gpus'] == 1 and d['steps'] == 1 and d['warmup'] == 0
  assert d['vs_baseline'] is None and d['data'] == 'synthetic' and d['dtype'] == 'f32'
  assert 'workload' in d['config'] and 'model' not in d['config']
  cb = d['cpu_baseline']
  assert cb['kind'] in ('reference', 'port') and cb['cores'] == 1 and cb['value'] == d['value'] and cb['sample']
  e2e = d['e2e']
  assert e2e['value'] == d['value'] and e2e['unit'] == d['unit']
  assert e2e['h2d_bytes_per_step'] == 0 and e2e['d2h_bytes_per_step'] == 0


@pytest.mark.skipif(torch.cuda.is_available(), reason='checks the behaviour on a machine without a GPU')
def test_own_arm_refuses_to_run_without_a_gpu():
  r = _run('--steps', '1', '--warmup', '0', timeout=120)
  assert r.returncode != 0
  assert 'CUDA device' in (r.stderr + r.stdout)
  assert not [l for l in r.stdout.splitlines() if l.startswith('{')]
