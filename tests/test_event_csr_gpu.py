"""GPU parity of event_csr_matvec / csr_matvec against the CPU oracle, the committed golden
outputs of the reference's CPU code and (when built) the reference's own CUDA kernels.

Tolerances (fp32): homogeneous weights in the scatter direction are bit-exact; homogeneous
weights in the gather direction are bit-exact against the oracle's float64 row accumulator;
everything else rtol 1e-5, atol 1e-5 * (largest row or column degree), allowing for the
order of atomic additions.
"""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden'))
import cases  # noqa: E402
import make_golden  # noqa: E402
import brainpylib_b200 as bpl  # noqa: E402
from brainpylib_b200 import gpu_ops, workloads  # noqa: E402
from oracle import cpu, ref  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'stored_matrix.npz'))


def dev(a, device):
  if isinstance(a, np.ndarray) and a.dtype == np.uint32:
    a = a.view(np.int32)
  return torch.as_tensor(a).to(device)


def atol_for(indptr, indices, n_col, transpose):
  if transpose:
    deg = np.bincount(indices, minlength=n_col).max() if indices.size else 1
  else:
    deg = np.diff(indptr).max() if indptr.size > 1 else 1
  return 1e-5 * max(int(deg), 1)


def run_event(device, data, indices, indptr, events, shape, transpose):
  y = bpl.event_csr_matvec(dev(data, device), dev(indices, device), dev(indptr, device), dev(events, device),
                           shape=shape, transpose=transpose)
  return y.cpu().numpy()


GOLD_EVENT = [c for c in make_golden.golden_cases() if c[1] in ('event_csr', 'c1')]
GOLD_CSR = [c for c in make_golden.golden_cases() if c[1] == 'csr']


@pytest.mark.parametrize('name,kind,kw', GOLD_EVENT, ids=[c[0] for c in GOLD_EVENT])
def test_event_csr_matches_reference_golden(cuda, name, kind, kw):
  inp = make_golden.build_inputs(kind, kw)
  x = inp['events'] if kind == 'c1' else inp['x']
  transpose = True if kind == 'c1' else inp['transpose']
  y = run_event(cuda, inp['data'], inp['indices'], inp['indptr'], x, inp['shape'], transpose)
  want = GOLDEN[name]
  if inp['data'].shape[0] == 1:
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32)), np.abs(y - want).max()
  else:
    np.testing.assert_allclose(y, want, rtol=1e-5,
                               atol=atol_for(inp['indptr'], inp['indices'], inp['shape'][1], transpose))


@pytest.mark.parametrize('name,kind,kw', GOLD_CSR, ids=[c[0] for c in GOLD_CSR])
def test_csr_matvec_matches_reference_golden(cuda, name, kind, kw):
  inp = make_golden.build_inputs(kind, kw)
  y = bpl.csr_matvec(dev(inp['data'], cuda), dev(inp['indices'], cuda), dev(inp['indptr'], cuda), dev(inp['x'], cuda),
                     shape=inp['shape'], transpose=inp['transpose']).cpu().numpy()
  np.testing.assert_allclose(y, GOLDEN[name], rtol=1e-5,
                             atol=atol_for(inp['indptr'], inp['indices'], inp['shape'][1], inp['transpose']))


@pytest.mark.parametrize('dtype', [np.float32, np.float64])
@pytest.mark.parametrize('ev_dtype', ['bool', 'same'])
@pytest.mark.parametrize('transpose', [True, False])
@pytest.mark.parametrize('homo', [True, False])
def test_event_csr_ragged_rows(cuda, dtype, ev_dtype, transpose, homo):
  """Empty rows, rows of 1/31/32/33/1000/5000 entries, duplicate columns, unaligned row starts."""
  rng = np.random.default_rng(11)
  lens = np.concatenate([[0, 1, 31, 32, 33, 1000, 0, 5000, 3, 0], rng.integers(0, 70, 300)])
  n_row, n_col = lens.shape[0], 1531
  data, indices, indptr, rng = cases.ragged_csr(lens, n_col, 12, dtype=dtype)
  if homo:
    data = np.array([0.6], dtype=dtype)
  n_in = n_row if transpose else n_col
  events = cases.events_like(rng, n_in, 0.3, np.bool_ if ev_dtype == 'bool' else dtype)
  if ev_dtype == 'same':
    events[events != 0] = rng.choice([1.0, 2.0, -3.5, np.nan], size=int((events != 0).sum()))  # truthiness only
  y = run_event(cuda, data, indices, indptr, events, (n_row, n_col), transpose)
  want = cpu.event_csr_matvec(data, indices, indptr, events, shape=(n_row, n_col), transpose=transpose)
  if homo and dtype == np.float32:
    assert y.tobytes() == want.tobytes()
  elif homo and transpose:
    assert y.tobytes() == want.tobytes()
  else:
    np.testing.assert_allclose(y, want, rtol=1e-5 if dtype == np.float32 else 1e-12,
                               atol=atol_for(indptr, indices, n_col, transpose))


@pytest.mark.parametrize('rate', [0.0, 1.0])
@pytest.mark.parametrize('transpose', [True, False])
def test_event_csr_no_events_and_all_events(cuda, rate, transpose):
  data, indices, indptr, rng = cases.csr_case((300, 500), 0.05, 21)
  n_in = 300 if transpose else 500
  events = np.full(n_in, rate == 1.0)
  y = run_event(cuda, data, indices, indptr, events, (300, 500), transpose)
  want = cpu.event_csr_matvec(data, indices, indptr, events, shape=(300, 500), transpose=transpose)
  np.testing.assert_allclose(y, want, rtol=1e-5, atol=atol_for(indptr, indices, 500, transpose))
  if rate == 0.0:
    assert not y.any()


@pytest.mark.parametrize('homo', [True, False])
@pytest.mark.parametrize('ev_dtype', [np.bool_, np.float32])
def test_event_csr_gather_with_shared_memory_event_mask(cuda, homo, ev_dtype):
  """Large enough (>= 4096 rows, >= 8192 columns) for the gather kernel that keeps the events as a
  bitmask in shared memory; a column count that is not a multiple of 32."""
  shape = (6000, 30011)
  data, indices, indptr, rng = cases.csr_case(shape, 0.004, 23, homo=0.6 if homo else None)
  for rate in (0.05, 1.0, 0.0):
    events = cases.events_like(rng, shape[1], rate, ev_dtype)
    y = run_event(cuda, data, indices, indptr, events, shape, False)
    want = cpu.event_csr_matvec(data, indices, indptr, events, shape=shape, transpose=False)
    if homo:
      assert y.tobytes() == want.tobytes()
    else:
      np.testing.assert_allclose(y, want, rtol=1e-5, atol=atol_for(indptr, indices, shape[1], False))


def test_event_csr_empty_matrix_and_tiny_shapes(cuda):
  for shape in [(1, 1), (1, 5), (5, 1), (3, 0), (0, 3)]:
    n_row, n_col = shape
    indptr = np.zeros(n_row + 1, dtype=np.int32)
    indices = np.zeros(0, dtype=np.int32)
    for transpose in (True, False):
      events = np.ones(n_row if transpose else n_col, dtype=np.bool_)
      y = run_event(cuda, np.array([1.], np.float32), indices, indptr, events, shape, transpose)
      assert y.shape == (n_col if transpose else n_row,) and not y.any()


def test_event_csr_unaligned_views(cuda):
  """Index / weight arrays that do not start on a 16-byte boundary take the element-wise path."""
  data, indices, indptr, rng = cases.csr_case((400, 300), 0.2, 31)
  events = rng.random(400) < 0.2
  want = cpu.event_csr_matvec(data, indices, indptr, events, shape=(400, 300), transpose=True)
  pad_i = torch.zeros(indices.shape[0] + 1, dtype=torch.int32, device=cuda)
  pad_d = torch.zeros(data.shape[0] + 1, dtype=torch.float32, device=cuda)
  pad_i[1:] = dev(indices, cuda)
  pad_d[1:] = dev(data, cuda)
  y = bpl.event_csr_matvec(pad_d[1:], pad_i[1:], dev(indptr, cuda), dev(events, cuda), shape=(400, 300),
                           transpose=True).cpu().numpy()
  np.testing.assert_allclose(y, want, rtol=1e-5, atol=atol_for(indptr, indices, 300, True))
  x = rng.uniform(-1, 1, 300).astype(np.float32)
  y = bpl.csr_matvec(pad_d[1:], pad_i[1:], dev(indptr, cuda), dev(x, cuda), shape=(400, 300)).cpu().numpy()
  np.testing.assert_allclose(y, cpu.csr_matvec(data, indices, indptr, x, shape=(400, 300)), rtol=1e-5, atol=1e-3)


def test_relations_of_the_reference_tests(cuda):
  """brainpylib/_src/event_ops/tests/test_event_csr_matvec.py:57-73: homo == heter with a constant,
  bool events == float events, == dense product."""
  for shape in cases.EVENT_CSR_SHAPES:
    for transpose in (True, False):
      for homo in (-1., 0., 1.):
        _, indices, indptr, rng = cases.csr_case(shape, 0.4, 41)
        events = rng.random(shape[0] if transpose else shape[1]) < 0.1
        d_idx, d_ptr, d_ev = dev(indices, cuda), dev(indptr, cuda), dev(events, cuda)
        r1 = bpl.event_csr_matvec(homo, d_idx, d_ptr, d_ev, shape=shape, transpose=transpose)
        heter = torch.full((indices.shape[0],), homo, dtype=torch.float32, device=cuda)
        r2 = bpl.event_csr_matvec(heter, d_idx, d_ptr, d_ev, shape=shape, transpose=transpose)
        assert torch.equal(r1, r2)   # integer-valued accumulation: exact in any order
        r3 = bpl.event_csr_matvec(homo, d_idx, d_ptr, d_ev.float(), shape=shape, transpose=transpose)
        assert torch.equal(r1, r3)
        r4 = bpl.cusparse_csr_matvec(torch.tensor([homo], device=cuda), d_idx, d_ptr, d_ev.float(), shape=shape,
                                     transpose=transpose)
        assert torch.equal(r1, r4)
        dense = bpl.csr_to_dense(torch.tensor([homo], device=cuda), d_idx, d_ptr, shape=shape)
        r5 = (d_ev.float() @ dense) if transpose else (dense @ d_ev.float())
        assert torch.equal(r1, r5)


def test_csr_methods_agree(cuda):
  c = workloads.config_c2(n=2000, degree=100)
  args = [dev(c[k], cuda) for k in ('data', 'indices', 'indptr', 'vector')]
  want = cpu.csr_matvec(c['data'], c['indices'], c['indptr'], c['vector'], shape=c['shape'])
  for method in ('scalar', 'vector', 'adaptive'):
    y = bpl.csr_matvec(*args, shape=c['shape'], method=method).cpu().numpy()
    np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-3)
  yt = bpl.csr_matvec(*args, shape=c['shape'], transpose=True).cpu().numpy()
  want_t = cpu.csr_matvec(c['data'], c['indices'], c['indptr'], c['vector'], shape=c['shape'], transpose=True)
  np.testing.assert_allclose(yt, want_t, rtol=1e-5, atol=atol_for(c['indptr'], c['indices'], 2000, True))


def test_twin_of_the_million_neuron_config(cuda):
  """1e5 neurons x 1000 synapses (1e8 nnz), unsorted columns with duplicates, U(0,1) weights,
  float32 events at 1 %: the CPU-checkable twin of the headline configuration."""
  c = workloads.config_c3_twin(n_steps=3)
  d = {k: dev(c[k], cuda) for k in ('data', 'indices', 'indptr')}
  for events in c['events']:
    y = bpl.event_csr_matvec(d['data'], d['indices'], d['indptr'], dev(events, cuda), shape=c['shape'],
                             transpose=True).cpu().numpy()
    want = cpu.event_csr_matvec(c['data'], c['indices'], c['indptr'], events, shape=c['shape'], transpose=True)
    np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-5 * 1000)
    # homogeneous twin: bit-exact
    yh = bpl.event_csr_matvec(0.6, d['indices'], d['indptr'], dev(events, cuda), shape=c['shape'],
                              transpose=True).cpu().numpy()
    wh = cpu.event_csr_matvec(np.float32(0.6), c['indices'], c['indptr'], events, shape=c['shape'], transpose=True)
    assert yh.tobytes() == wh.tobytes()


needs_ref_gpu = pytest.mark.skipif(not ref.available_gpu(), reason='oracle/_ref/libref_gpu.so not built')


@needs_ref_gpu
@pytest.mark.parametrize('transpose', [True, False])
@pytest.mark.parametrize('homo', [True, False])
def test_against_reference_cuda_kernels(cuda, transpose, homo):
  """Same inputs through the reference's own kernels (lib/gpu_event_csr_matvec.cu, lib/gpu_csr_matvec.cu)."""
  shape = (3000, 2000)
  data, indices, indptr, rng = cases.csr_case(shape, 0.05, 51, homo=3.0 if homo else None)
  events = (rng.random(shape[0] if transpose else shape[1]) < 0.1).astype(np.float32)
  t = [dev(a, cuda) for a in (data, indices, indptr, events)]
  y = bpl.event_csr_matvec(*t, shape=shape, transpose=transpose)
  y_ref = torch.empty_like(y)
  name = 'event_csr_matvec_' + ('homo' if homo else 'heter') + '_float_float'
  ref.gpu_call(name, t + [y_ref], gpu_ops.build_twouint_onebool_descriptor(shape[0], shape[1], transpose))
  if homo:
    assert torch.equal(y, y_ref)
  else:
    torch.testing.assert_close(y, y_ref, rtol=1e-5, atol=atol_for(indptr, indices, shape[1], transpose))
  if not transpose:
    x = dev(rng.uniform(-1, 1, shape[1]).astype(np.float32), cuda)
    y = bpl.csr_matvec(t[0], t[1], t[2], x, shape=shape)
    y_ref = torch.empty_like(y)
    name = 'csr_matvec_' + ('homo' if homo else 'heter') + '_vector_float'
    ref.gpu_call(name, [t[0], t[1], t[2], x, y_ref], gpu_ops.build_double_size_descriptor(*shape))
    torch.testing.assert_close(y, y_ref, rtol=1e-5, atol=1e-3)


def test_gradients_follow_the_reference_rules(cuda):
  """brainpylib/_src/event_ops/event_csr_matvec.py:439-463 via torch autograd, against a dense matrix."""
  shape = (60, 80)
  data, indices, indptr, rng = cases.csr_case(shape, 0.3, 61, dtype=np.float64)
  for transpose in (True, False):
    n_in = shape[0] if transpose else shape[1]
    ev = torch.as_tensor((rng.random(n_in) < 0.4).astype(np.float64), device=cuda).requires_grad_(True)
    w = dev(data, cuda).requires_grad_(True)
    idx, ptr = dev(indices, cuda), dev(indptr, cuda)
    ct = torch.as_tensor(rng.standard_normal(shape[1] if transpose else shape[0]), device=cuda)
    y = bpl.event_csr_matvec(w, idx, ptr, ev, shape=shape, transpose=transpose)
    gw, gev = torch.autograd.grad(y, (w, ev), ct)
    w2 = dev(data, cuda).requires_grad_(True)
    ev2 = ev.detach().clone().requires_grad_(True)
    dense = bpl.csr_to_dense(w2, idx, ptr, shape=shape)
    y2 = (ev2 @ dense) if transpose else (dense @ ev2)
    gw2, gev2 = torch.autograd.grad(y2, (w2, ev2), ct)
    torch.testing.assert_close(y, y2, rtol=1e-10, atol=1e-10)
    torch.testing.assert_close(gw, gw2, rtol=1e-10, atol=1e-10)
    torch.testing.assert_close(gev, gev2, rtol=1e-10, atol=1e-10)
    # homogeneous weight
    wh = torch.tensor([0.7], dtype=torch.float64, device=cuda, requires_grad=True)
    yh = bpl.event_csr_matvec(wh, idx, ptr, ev.detach(), shape=shape, transpose=transpose)
    gh, = torch.autograd.grad(yh, wh, ct)
    ones = bpl.csr_to_dense(torch.ones(1, dtype=torch.float64, device=cuda), idx, ptr, shape=shape)
    r = (ev.detach() @ ones) if transpose else (ones @ ev.detach())
    torch.testing.assert_close(gh, torch.dot(ct, r).reshape(1), rtol=1e-10, atol=1e-10)
