"""Known-answer tests of the just-in-time-connectivity path against outputs of the REFERENCE's own
CUDA kernels (tests/golden/jitconn_reference_gpu.npz, made on a B200 by
tests/golden/make_golden_jitconn.py from lib/gpu_jitconn_*.cu).

* not gpu: the CPU oracle (oracle/jitconn_oracle.cu: cuRAND's header compiled for the host) must
  reproduce them.  Host and device `logf` differ in the last bit for some arguments, which moves a
  sampled position by one where the quotient sits next to an integer; the oracle counts those draws
  ("fragile") and at most that many outputs may differ.  Host `curand_normal` uses sinf/cosf where
  the device uses __sincosf, so normal weights are compared at 1e-4 relative.
* gpu: this library's kernels must reproduce them bit for bit wherever the order of additions is
  fixed (row-parallel ops, matmat, homogeneous column-parallel event ops), else within 1e-5.
"""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden'))
import make_golden_jitconn as mg  # noqa: E402
from oracle import cpu  # noqa: E402

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'jitconn_reference_gpu.npz'))
CASES = mg.jitconn_cases()
ORACLE_KIND = {'homo': cpu.W_HOMO, 'uniform': cpu.W_UNIFORM, 'normal': cpu.W_NORMAL}


def test_every_jitconn_golden_case_is_stored():
  assert sorted(GOLDEN.files) == sorted(n for n, _ in CASES)


@pytest.mark.parametrize('name,spec', CASES, ids=[c[0] for c in CASES])
def test_cpu_oracle_matches_reference_gpu_golden(name, spec):
  x = mg.case_inputs(spec)
  kw = dict(kind=ORACLE_KIND[spec['kind']], w1=spec['w1'], w2=spec['w2'], conn_prob=spec['prob'], shape=spec['shape'],
            seed=spec['seed'], return_info=True)
  if spec['op'] == 'event':
    y, info = cpu.jitconn_event_matvec(x, outdim_parallel=spec['odp'], **kw)
  elif spec['op'] == 'matvec':
    y, info = cpu.jitconn_matvec(x, outdim_parallel=spec['odp'], **kw)
  else:
    y, info = cpu.jitconn_matmat(x, **kw)
  want = GOLDEN[name]
  assert y.shape == want.shape
  rtol = 1e-4 if spec['kind'] == 'normal' else 2e-5
  scale = max(1.0, float(np.abs(want).max()))
  bad = ~np.isclose(y, want, rtol=rtol, atol=2e-6 * scale)
  if spec['op'] == 'matmat':
    bad = bad.any(axis=0)          # a moved position changes a whole output column
  # a fragile draw moves one synapse: it changes one output of a row-parallel op, at most two
  # outputs of a column-parallel one
  assert int(bad.sum()) <= 2 * info['fragile'], (int(bad.sum()), info)


@pytest.mark.gpu
@pytest.mark.parametrize('name,spec', CASES, ids=[c[0] for c in CASES])
def test_kernels_match_reference_gpu_golden(cuda, name, spec):
  import torch
  from brainpylib_b200 import jitconn_ops
  x = torch.as_tensor(mg.case_inputs(spec)).to(cuda)
  kw = dict(kind=spec['kind'], w1=spec['w1'], w2=spec['w2'], conn_prob=spec['prob'], shape=spec['shape'], seed=spec['seed'])
  if spec['op'] == 'event':
    y = jitconn_ops.event_matvec_raw(x, transpose=False, outdim_parallel=spec['odp'], **kw)
  elif spec['op'] == 'matvec':
    y = jitconn_ops.matvec_raw(x, transpose=False, outdim_parallel=spec['odp'], **kw)
  else:
    y = jitconn_ops.matmat_raw(x, **kw)
  y = y.cpu().numpy()
  want = GOLDEN[name]
  ordered = spec['op'] == 'matmat' or spec['odp'] or (spec['op'] == 'event' and spec['kind'] == 'homo')
  if ordered:
    assert y.tobytes() == want.tobytes(), np.abs(y - want).max()
  else:
    np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-5 * max(1.0, spec['prob'] * spec['shape'][1]))
