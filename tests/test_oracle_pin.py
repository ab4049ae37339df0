"""Pins the CPU oracle (oracle/liboracle.so) to the reference:

* against the committed golden outputs of the reference's own CPU code
  (tests/golden/stored_matrix.npz, made by tests/golden/make_golden.py), and
* live against oracle/_ref/libref_cpu.so and the reference's numba kernels when the
  reference tree / the prebuilt library is present.

Tolerances: transposed (scatter) products are bit-exact (same serial order); gather
products with a float64 row accumulator are bit-exact too; the transposed dense product
is compared with rtol 1e-5 because the reference's numba kernel (fastmath) may fuse the
multiply-add while the oracle rounds the product first, as a GPU atomic scatter does.
"""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden'))
import make_golden  # noqa: E402
from oracle import cpu, ref  # noqa: E402

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'stored_matrix.npz'))
CASES = make_golden.golden_cases()


def oracle_output(kind, inp):
  if kind == 'c1':
    return cpu.event_csr_matvec(inp['data'], inp['indices'], inp['indptr'], inp['events'],
                                shape=inp['shape'], transpose=True)
  if kind == 'event_csr':
    return cpu.event_csr_matvec(inp['data'], inp['indices'], inp['indptr'], inp['x'],
                                shape=inp['shape'], transpose=inp['transpose'])
  if kind in ('csr', 'c2'):
    return cpu.csr_matvec(inp['data'], inp['indices'], inp['indptr'], inp['x'],
                          shape=inp['shape'], transpose=inp['transpose'])
  if kind == 'c3':
    return cpu.event_csr_matvec(inp['data'], inp['indices'], inp['indptr'], inp['x'], shape=inp['shape'], transpose=True)
  fn = cpu.coo_atomic_sum if inp['op'] == 'sum' else cpu.coo_atomic_prod
  return fn(inp['values'], inp['post'], inp['post_num'], None if inp['homo'] else inp['pre'])


def test_every_golden_case_is_stored():
  assert sorted(GOLDEN.files) == sorted(name for name, _, _ in CASES)


@pytest.mark.parametrize('name,kind,kw', CASES, ids=[c[0] for c in CASES])
def test_oracle_matches_golden(name, kind, kw):
  inp = make_golden.build_inputs(kind, kw)
  y = oracle_output(kind, inp)
  if 'stride' in kw:          # benchmark-size cases are stored as strided samples
    y = y[::kw['stride']]
  want = GOLDEN[name]
  assert y.shape == want.shape and y.dtype == want.dtype
  if kind == 'c2' and not kw['transpose']:
    # 100-term float32 rows: the reference's numba kernel may keep the row sum in a wider register
    np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-5)
  elif kind in ('csr', 'c2') and kw['transpose']:
    np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-5)
  else:
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32)), np.abs(y - want).max()


needs_ref = pytest.mark.skipif(not ref.available_cpu(), reason='oracle/_ref/libref_cpu.so not built')
needs_tree = pytest.mark.skipif(not os.path.isdir(os.path.join(ref.REFERENCE_ROOT, 'brainpylib')),
                                reason='reference tree not mounted')


@needs_ref
@pytest.mark.parametrize('dtype', [np.float32, np.float64])
@pytest.mark.parametrize('homo', [True, False])
def test_oracle_matches_live_reference_cpp(dtype, homo):
  rng = np.random.default_rng(7)
  lens = np.concatenate([[0, 1, 31, 32, 33, 1000, 0], rng.integers(0, 80, 500)])
  import cases
  data, indices, indptr, rng = cases.ragged_csr(lens, 777, 8, dtype=dtype)
  if homo:
    data = np.array([0.6], dtype=dtype)
  events = rng.random(lens.shape[0]) < 0.3
  want = ref.csr_event_sum(events, indices, indptr, data, 777)
  got = cpu.event_csr_matvec(data, indices, indptr, events, shape=(lens.shape[0], 777), transpose=True)
  assert got.tobytes() == want.tobytes()


@needs_tree
def test_oracle_matches_live_numba_twin_slice():
  """A slice of the reduced twin of the 1e6-neuron configuration: unsorted columns with duplicates."""
  from brainpylib_b200 import workloads
  rng = np.random.default_rng(3)
  n, deg = 5000, 1000
  indices = rng.integers(0, n, size=n * deg, dtype=np.int32)
  data = rng.random(n * deg, dtype=np.float32)
  indptr = np.arange(0, n * deg + 1, deg, dtype=np.int32)
  events = workloads.c3_events(rng, n, 0.01)
  want = ref.numba_event_csr_matvec(data, indices, indptr, events, shape=(n, n), transpose=True)
  got = cpu.event_csr_matvec(data, indices, indptr, events, shape=(n, n), transpose=True)
  assert got.tobytes() == want.tobytes()
  assert cpu.count_active_synapses(indptr, events) == int(events.sum()) * deg


def test_jitconn_oracle_relations():
  """The relations the reference's own jitconn tests assert (brainpylib/_src/jitconn_ops/tests/
  test_event_matvec.py:63-87, matmat_testcase.py:59-78), applied to the oracle."""
  rng = np.random.default_rng(0)
  shape, p, seed = (100, 200), 0.1, 1234
  ev = rng.random(200) < 0.3
  for kind, w1, w2 in ((cpu.W_HOMO, 0, 0), (cpu.W_UNIFORM, -0.1, 0.2), (cpu.W_NORMAL, 0., 0.01)):
    a = cpu.jitconn_event_matvec(ev, kind=kind, w1=w1, w2=w2, conn_prob=p, shape=shape, seed=seed)
    b = cpu.jitconn_event_matvec(ev, kind=kind, w1=w1, w2=w2, conn_prob=p, shape=shape, seed=seed)
    assert a.tobytes() == b.tobytes()                       # deterministic
    c = cpu.jitconn_event_matvec(ev, kind=kind, w1=w1, w2=w2, conn_prob=p, shape=shape[::-1], seed=seed,
                                 transpose=True)
    assert a.tobytes() == c.tobytes()                       # (shape, T) == (shape[::-1], not T)
    # row-parallel M and column-parallel M^T walk the same streams: <M x, z> == <x, M^T z>
    x = rng.standard_normal(200).astype(np.float32)
    z = rng.standard_normal(100).astype(np.float32)
    mx = cpu.jitconn_matvec(x, kind=kind, w1=w1, w2=w2, conn_prob=p, shape=shape, seed=seed)
    mtz = cpu.jitconn_matvec(z, kind=kind, w1=w1, w2=w2, conn_prob=p, shape=shape, seed=seed, transpose=True,
                             outdim_parallel=False)
    np.testing.assert_allclose(np.dot(mx.astype(np.float64), z), np.dot(x.astype(np.float64), mtz), rtol=1e-4)
    # event product with float events == dense product for weighted kinds
    evf = ev.astype(np.float32)
    d = cpu.jitconn_matvec(evf, kind=kind, w1=w1, w2=w2, conn_prob=p, shape=shape, seed=seed)
    np.testing.assert_allclose(a, d, rtol=1e-5, atol=1e-6)
  # matmat == matvec(transpose=True) row by row
  X = rng.standard_normal((5, 100)).astype(np.float32)
  Y = cpu.jitconn_matmat(X, kind=cpu.W_NORMAL, w1=0., w2=0.01, conn_prob=p, shape=shape, seed=seed)
  for r in range(5):
    yr = cpu.jitconn_matvec(X[r], kind=cpu.W_NORMAL, w1=0., w2=0.01, conn_prob=p, shape=shape, seed=seed,
                            transpose=True)
    assert Y[r].tobytes() == yr.tobytes()


def test_jitconn_stream_statistics():
  """Gaps are geometric: about p * extent connections per stream, positions strictly inside the extent."""
  pos, w, fragile = cpu.jitconn_stream(42, conn_prob=0.01, extent=100000, kind=cpu.W_UNIFORM, w1=-0.1, w2=0.2)
  assert 800 < pos.shape[0] < 1200
  assert pos.min() >= 0 and pos.max() < 100000 and np.all(np.diff(pos) >= 0)
  assert w.min() >= -0.1 and w.max() <= 0.1
  assert fragile <= 2
