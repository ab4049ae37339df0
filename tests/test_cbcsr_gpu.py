"""GPU parity of the column-blocked CSR format and its transposed event product against the CPU
oracle of the plain CSR operator (same matrix, same events): rtol 1e-5, atol 1e-5 * largest in-degree
(the additions of one output neuron are grouped by CTA and may come in any order)."""
import numpy as np
import pytest
import torch

import cases
import brainpylib_b200 as bpl
from brainpylib_b200 import event_ops, workloads
from oracle import cpu

pytestmark = pytest.mark.gpu


def check(cuda, data, indices, indptr, shape, events_list, block_width=None, rows_per_pass=100_000):
  t = [torch.as_tensor(a).to(cuda) for a in (data, indices, indptr)]
  cb = bpl.csr_to_column_blocked(*t, shape=shape, block_width=block_width, rows_per_pass=rows_per_pass)
  assert int(cb.offsets[-1, -1]) == indices.shape[0] and int(cb.offsets[0, 0]) == 0
  atol = 1e-5 * max(1, int(np.bincount(indices, minlength=shape[1]).max())) if indices.size else 1e-5
  for ev in events_list:
    y = bpl.event_cbcsr_matvec(cb, torch.as_tensor(ev).to(cuda)).cpu().numpy()
    want = cpu.event_csr_matvec(data, indices, indptr, ev, shape=shape, transpose=True)
    np.testing.assert_allclose(y, want, rtol=1e-5, atol=atol)
  return cb


@pytest.mark.parametrize('shape', cases.EVENT_CSR_SHAPES + [(3000, 5000), (5000, 70001)])
def test_cbcsr_matches_oracle(cuda, shape):
  prob = 0.4 if shape[0] * shape[1] < 1e6 else 0.01
  data, indices, indptr, rng = cases.csr_case(shape, prob, 81)
  evs = [rng.random(shape[0]) < r for r in (0.1, 0.0, 1.0)]
  evs.append((rng.random(shape[0]) < 0.3).astype(np.float32) * 2.5)
  check(cuda, data, indices, indptr, shape, evs)
  check(cuda, data, indices, indptr, shape, evs[:1], block_width=1024, rows_per_pass=977)


def test_cbcsr_long_segments_duplicates_and_ragged_rows(cuda):
  """Rows of 0 / 1 / 33 / 5000 entries into 300 columns: segments far longer than a warp, duplicates."""
  rng = np.random.default_rng(82)
  lens = np.concatenate([[0, 1, 31, 32, 33, 5000, 0, 700], rng.integers(0, 90, 200)])
  data, indices, indptr, rng = cases.ragged_csr(lens, 300, 83)
  evs = [rng.random(lens.shape[0]) < r for r in (0.5, 1.0)]
  check(cuda, data, indices, indptr, (lens.shape[0], 300), evs, block_width=128)
  check(cuda, data, indices, indptr, (lens.shape[0], 300), evs)


def test_cbcsr_twin_of_the_million_neuron_config(cuda):
  c = workloads.config_c3_twin(n_steps=2)
  cb = check(cuda, c['data'], c['indices'], c['indptr'], c['shape'], c['events'])
  assert cb.n_blocks == -(-c['shape'][1] // cb.block_width)
  # 6 bytes per synapse + the per-row block offsets
  assert cb.nbytes() == 6 * c['data'].shape[0] + 4 * (cb.n_blocks + 1) * c['shape'][0]


def test_cbcsr_empty_and_errors(cuda):
  indptr = np.zeros(6, dtype=np.int32)
  cb = bpl.csr_to_column_blocked(torch.zeros(0, device=cuda), torch.zeros(0, dtype=torch.int32, device=cuda),
                                 torch.as_tensor(indptr).to(cuda), shape=(5, 7))
  y = bpl.event_cbcsr_matvec(cb, torch.ones(5, dtype=torch.bool, device=cuda))
  assert y.shape == (7,) and not y.any()
  with pytest.raises(ValueError):
    bpl.event_cbcsr_matvec(cb, torch.ones(4, dtype=torch.bool, device=cuda))
  with pytest.raises(ValueError):
    bpl.csr_to_column_blocked(torch.zeros(0, device=cuda), torch.zeros(0, dtype=torch.int32, device=cuda),
                              torch.as_tensor(indptr).to(cuda), shape=(5, 7), block_width=70000)
