"""GPU parity of the column-blocked format: the CUDA builder against the numpy statement of the layout
(byte for byte), and the transposed event product on it against the CPU oracle of the plain CSR operator
(same matrix, same events): rtol 1e-5, atol 1e-5 * largest in-degree (the additions of one output neuron
are grouped by CTA and may come in any order)."""
import numpy as np
import pytest
import torch

import cases
import brainpylib_b200 as bpl
from brainpylib_b200 import event_ops, workloads
from oracle import cpu

pytestmark = pytest.mark.gpu


def build(cuda, data, indices, indptr, shape, block_width=None, col_range=None, compare_layout=True, accumulate='float'):
  t = [torch.as_tensor(a).to(cuda) for a in (data, indices, indptr)]
  cb = bpl.csr_to_column_blocked(*t, shape=shape, block_width=block_width, col_range=col_range, accumulate=accumulate)
  if compare_layout:
    groups, offsets = cases.column_blocked_model(data, indices, indptr, shape[1], cb.block_width, col_range)
    np.testing.assert_array_equal(cb.offsets.cpu().numpy().view(np.uint32), offsets)
    assert cb.groups.cpu().numpy().tobytes() == groups.tobytes()
  return cb


def check(cuda, data, indices, indptr, shape, events_list, block_width=None, compare_layout=True):
  """Both accumulation modes against the oracle.  Fixed point: every weight is rounded to a multiple of 2^-k, so an
  output is off by at most (its in-degree) * 2^-(k+1) on top of nothing else; that bound is added to the tolerance."""
  cb = None
  for accumulate in ('float', 'fixed'):
    cb = build(cuda, data, indices, indptr, shape, block_width, compare_layout=compare_layout and accumulate == 'float',
               accumulate=accumulate)
    deg = max(1, int(np.bincount(indices, minlength=shape[1]).max())) if indices.size else 1
    atol = 1e-5 * deg
    if accumulate == 'fixed':
      col_abs = np.zeros(shape[1])
      np.add.at(col_abs, indices, np.abs(np.broadcast_to(data, indices.shape) if data.shape[0] == 1 else data))
      assert cb.scale_log2 == event_ops.fixed_point_scale_log2(float(np.float32(col_abs.max()))) or \
          abs(cb.scale_log2 - event_ops.fixed_point_scale_log2(float(col_abs.max()))) <= 1
      atol += deg * 2.0 ** -(cb.scale_log2 + 1)
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
  small = shape[0] * shape[1] < 3e6
  check(cuda, data, indices, indptr, shape, evs, compare_layout=small)
  check(cuda, data, indices, indptr, shape, evs[:1], block_width=1024, compare_layout=small)


def test_cbcsr_long_segments_duplicates_and_ragged_rows(cuda):
  """Rows of 0 / 1 / 33 / 5000 entries into 300 columns: segments that fill several ring stages, duplicates."""
  rng = np.random.default_rng(82)
  lens = np.concatenate([[0, 1, 31, 32, 33, 5000, 0, 700, 20000], rng.integers(0, 90, 200)])
  data, indices, indptr, rng = cases.ragged_csr(lens, 300, 83)
  evs = [rng.random(lens.shape[0]) < r for r in (0.5, 1.0)]
  check(cuda, data, indices, indptr, (lens.shape[0], 300), evs, block_width=128)
  check(cuda, data, indices, indptr, (lens.shape[0], 300), evs)


def test_cbcsr_widest_block_and_many_rows_per_warp(cuda):
  """70000 active rows over 2 column blocks of the largest width = 16 CTA shares of 4375 rows: every warp walks several
  batches of 32 rows with only two ring buffers (the slice takes most of the shared memory)."""
  shape = (70000, 40000)
  rng = np.random.default_rng(84)
  lens = rng.integers(10, 30, shape[0])
  data, indices, indptr, rng = cases.ragged_csr(lens, shape[1], 84)
  check(cuda, data, indices, indptr, shape, [np.ones(shape[0], dtype=bool)], block_width=32256, compare_layout=False)


def test_cbcsr_homogeneous_weight_and_column_range(cuda):
  shape = (300, 1000)
  data, indices, indptr, rng = cases.csr_case(shape, 0.05, 85, homo=0.6)
  cb = build(cuda, data, indices, indptr, shape, block_width=64, col_range=(250, 700))
  assert cb.shape == (300, 450) and cb.col_range == (250, 700)
  ev = rng.random(300) < 0.3
  y = bpl.event_cbcsr_matvec(cb, torch.as_tensor(ev).to(cuda)).cpu().numpy()
  want = cpu.event_csr_matvec(data, indices, indptr, ev, shape=shape, transpose=True)[250:700]
  np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-4)


def test_cbcsr_twin_of_the_million_neuron_config(cuda):
  c = workloads.config_c3_twin(n_steps=2)
  cb = check(cuda, c['data'], c['indices'], c['indptr'], c['shape'], c['events'], compare_layout=False)
  assert cb.n_blocks == -(-c['shape'][1] // cb.block_width)
  # the public operator takes the prepared matrix
  t = [torch.as_tensor(c[k]).to(cuda) for k in ('data', 'indices', 'indptr')]
  ev = torch.as_tensor(c['events'][0]).to(cuda)
  y0 = bpl.event_csr_matvec(*t, ev, shape=c['shape'], transpose=True)
  y1 = bpl.event_csr_matvec(*t, ev, shape=c['shape'], transpose=True, prepared=cb)
  torch.testing.assert_close(y1, y0, rtol=1e-5, atol=1e-2)
  assert not torch.equal(y1, torch.zeros_like(y1))


def test_cbcsr_empty_and_errors(cuda):
  indptr = np.zeros(6, dtype=np.int32)
  cb = bpl.csr_to_column_blocked(torch.zeros(0, device=cuda), torch.zeros(0, dtype=torch.int32, device=cuda),
                                 torch.as_tensor(indptr).to(cuda), shape=(5, 7))
  assert cb.n_groups == 0
  y = bpl.event_cbcsr_matvec(cb, torch.ones(5, dtype=torch.bool, device=cuda))
  assert y.shape == (7,) and not y.any()
  with pytest.raises(ValueError):
    bpl.event_cbcsr_matvec(cb, torch.ones(4, dtype=torch.bool, device=cuda))
  for bad in (70000, 33, 0):
    with pytest.raises(ValueError):
      bpl.csr_to_column_blocked(torch.zeros(0, device=cuda), torch.zeros(0, dtype=torch.int32, device=cuda),
                                torch.as_tensor(indptr).to(cuda), shape=(5, 7), block_width=bad)


@pytest.mark.parametrize('transpose', [True, False])
@pytest.mark.parametrize('shape,density,width', [((3000, 2000), 0.02, 512), ((20000, 50000), 0.002, None),
                                                 ((1, 40), 1.0, 32), ((700, 33000), 0.01, 32256)])
def test_dense_vector_product_on_the_prepared_matrix(cuda, shape, density, width, transpose):
  """csr_matvec(..., prepared=P) in both orientations with a dense x, against the CPU oracle and the stateless
  operator (float32 summation order differs: rtol 1e-5, atol 1e-5 * entries per output), zeros in x skipped, and the
  vector's tangent / cotangent rules against dense algebra."""
  import brainpylib_b200 as bpl
  from oracle import cpu
  data, indices, indptr, rng = cases.csr_case(shape, density, 31)
  n_in, n_out = (shape[0], shape[1]) if transpose else (shape[1], shape[0])
  x = rng.uniform(-1, 1, n_in).astype(np.float32)
  x[rng.random(n_in) < 0.3] = 0.0
  d, ix, ptr, xv = (torch.as_tensor(a).to(cuda) for a in (data, indices, indptr, x))
  prepared = bpl.csr_to_column_blocked(d, ix, ptr, shape=shape, block_width=width)
  y = bpl.csr_matvec(d, ix, ptr, xv, shape=shape, transpose=transpose, prepared=prepared)
  want = cpu.csr_matvec(data, indices, indptr, x, shape=shape, transpose=transpose)
  per_out = max(1.0, len(indices) / n_out)
  np.testing.assert_allclose(y.cpu().numpy(), want, rtol=1e-5, atol=1e-5 * per_out)
  plain = bpl.csr_matvec(d, ix, ptr, xv, shape=shape, transpose=transpose)
  torch.testing.assert_close(y, plain, rtol=1e-5, atol=1e-5 * per_out)
  if shape[0] * shape[1] <= 10_000_000:
    dense = bpl.sparse_ops.csr_to_dense(d, ix, ptr, shape=shape)
    op = dense.T if transpose else dense
    xg = xv.clone().requires_grad_(True)
    out = bpl.csr_matvec(d, ix, ptr, xg, shape=shape, transpose=transpose, prepared=prepared)
    ct = torch.as_tensor(rng.standard_normal(n_out).astype(np.float32)).to(cuda)
    out.backward(ct)
    torch.testing.assert_close(xg.grad, op.T @ ct, rtol=1e-4, atol=1e-4 * per_out)
    t = torch.as_tensor(rng.standard_normal(n_in).astype(np.float32)).to(cuda)
    _, tangent = torch.func.jvp(lambda v: bpl.csr_matvec(d, ix, ptr, v, shape=shape, transpose=transpose, prepared=prepared),
                                (xv,), (t,))
    torch.testing.assert_close(tangent, op @ t, rtol=1e-4, atol=1e-4 * per_out)


def test_dense_vector_product_refuses_fixed_point_and_wrong_operands(cuda):
  import brainpylib_b200 as bpl
  data, indices, indptr, rng = cases.csr_case((500, 400), 0.05, 3)
  d, ix, ptr = (torch.as_tensor(a).to(cuda) for a in (data, indices, indptr))
  x = torch.ones(500, device=cuda)
  fixed = bpl.csr_to_column_blocked(d, ix, ptr, shape=(500, 400), block_width=128, accumulate='fixed')
  with pytest.raises(ValueError, match='float'):
    bpl.csr_matvec(d, ix, ptr, x, shape=(500, 400), transpose=True, prepared=fixed)
  other = bpl.csr_to_column_blocked(d, ix, ptr, shape=(500, 400), block_width=128)
  other.shape = (500, 401)
  with pytest.raises(ValueError, match='prepared matrix has shape'):
    bpl.csr_matvec(d, ix, ptr, x, shape=(500, 400), transpose=True, prepared=other)
