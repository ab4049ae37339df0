"""Parity at the sizes the benchmark configurations are quoted on.

C2 (1e5 x 1e5, 100 entries per row, both orientations) is compared in full with the CPU oracle and with
the stored sample of the reference's numba kernels.  C3 (1e6 neurons x 1000 synapses) does not fit a CPU
check in full, so two steps are run on the whole 1e9-synapse matrix with the spikes outside pre-synaptic
rows 0..99,999 cleared and compared with the oracle (and the stored sample of the reference's C++ kernel)
on those rows; an unmasked step is then checked through properties that need no CPU pass over the
matrix: the two storage formats agree, and the sum of the output equals the sum of the active rows'
weights.  Tolerances: rtol 1e-5, atol 1e-5 * largest degree (fp32, atomics in any order).
"""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden'))
import make_golden  # noqa: E402
import brainpylib_b200 as bpl  # noqa: E402
from brainpylib_b200 import event_ops, workloads  # noqa: E402
from oracle import cpu  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'stored_matrix.npz'))


@pytest.mark.parametrize('transpose', [False, True])
def test_c2_full_size_against_oracle_and_reference_sample(cuda, transpose):
  c = workloads.config_c2()
  args = [torch.as_tensor(c[k]).to(cuda) for k in ('data', 'indices', 'indptr', 'vector')]
  y = bpl.csr_matvec(*args, shape=c['shape'], transpose=transpose).cpu().numpy()
  want = cpu.csr_matvec(c['data'], c['indices'], c['indptr'], c['vector'], shape=c['shape'], transpose=transpose)
  deg = int(np.bincount(c['indices'], minlength=c['shape'][1]).max()) if transpose else 100
  np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-5 * deg)
  kw = dict(transpose=transpose, stride=49)
  np.testing.assert_allclose(y[::49], GOLDEN[f'csr/C2/T{int(transpose)}'], rtol=1e-5, atol=1e-5 * deg)
  assert ('csr/C2/T%d' % transpose, 'c2', kw) in make_golden.golden_cases()


@pytest.fixture(scope='module')
def c3_on_device(cuda):
  n = 1_000_000
  parts = {'indices': [], 'data': []}
  for kind, c, arr in workloads.c3_matrix_chunks(n):
    if kind != 'rng':
      parts[kind].append(torch.from_numpy(arr).to(cuda))
  indices, data = torch.cat(parts['indices']), torch.cat(parts['data'])
  del parts
  indptr = torch.arange(0, n * 1000 + 1, 1000, dtype=torch.int32, device=cuda)
  yield dict(indices=indices, data=data, indptr=indptr, shape=(n, n))
  del indices, data
  torch.cuda.empty_cache()


def test_c3_full_size_two_steps_against_oracle(cuda, c3_on_device):
  m = c3_on_device
  rows = workloads.config_c3_first_rows(2)
  assert torch.equal(m['indices'][:rows['indices'].shape[0]].cpu(), torch.from_numpy(rows['indices']))
  prepared = bpl.prepare_event_csr(m['data'], m['indices'], m['indptr'], shape=m['shape'])
  heter_atol = 1e-2            # 1e-5 * nnz per row (1000), the tolerance stated for this configuration
  for step in range(2):
    ev = rows['events_masked'][step]
    want = cpu.event_csr_matvec(rows['data'], rows['indices'], rows['indptr'], ev[:rows['shape'][0]],
                                shape=rows['shape'], transpose=True)
    d_ev = torch.from_numpy(ev).to(cuda)
    y = bpl.event_csr_matvec(m['data'], m['indices'], m['indptr'], d_ev, shape=m['shape'], transpose=True)
    np.testing.assert_allclose(y.cpu().numpy(), want, rtol=1e-5, atol=heter_atol)
    np.testing.assert_allclose(y.cpu().numpy()[::499], GOLDEN[f'event_csr/C3_rows_0_99999/step{step}'], rtol=1e-5,
                               atol=heter_atol)
    yp = bpl.event_csr_matvec(m['data'], m['indices'], m['indptr'], d_ev, shape=m['shape'], transpose=True,
                              prepared=prepared)
    np.testing.assert_allclose(yp.cpu().numpy(), want, rtol=1e-5, atol=heter_atol)
    # homogeneous weight 0.6 on the same connectivity: bit-exact against the serial sum
    homo = torch.tensor([0.6], device=cuda)
    yh = bpl.event_csr_matvec(homo, m['indices'], m['indptr'], d_ev, shape=m['shape'], transpose=True)
    want_h = cpu.event_csr_matvec(np.array([0.6], np.float32), rows['indices'], rows['indptr'],
                                  ev[:rows['shape'][0]], shape=rows['shape'], transpose=True)
    assert yh.cpu().numpy().tobytes() == want_h.tobytes()
  # one unmasked step (about 1e7 synapses): format agreement and the checksum of the active rows
  ev = torch.from_numpy(rows['events'][0]).to(cuda)
  y = bpl.event_csr_matvec(m['data'], m['indices'], m['indptr'], ev, shape=m['shape'], transpose=True)
  yp = bpl.event_csr_matvec(m['data'], m['indices'], m['indptr'], ev, shape=m['shape'], transpose=True,
                            prepared=prepared)
  torch.testing.assert_close(yp, y, rtol=1e-5, atol=heter_atol)
  active = torch.nonzero(ev).flatten()
  row_sums = m['data'].view(-1, 1000)[active].double().sum()
  assert abs(y.double().sum().item() - row_sums.item()) < 1e-6 * row_sums.item()
  assert abs(yp.double().sum().item() - row_sums.item()) < 1e-6 * row_sums.item()
