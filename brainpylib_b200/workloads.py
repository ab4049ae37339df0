"""Seeded synthetic inputs for the benchmark configurations and the small test shapes.

All draws use ``numpy.random.Generator(PCG64)`` in the order written here, so the
same inputs can be rebuilt anywhere from the seed alone.  They stand in for the
spike trains and connectivity a simulator would produce (the COBA E/I network of
brainpylib/_src/op_register/tests/ei_net.py:57-72 gives C1 its shape).
"""
import numpy as np

__all__ = [
  'fixed_prob_csr', 'fixed_degree_csr', 'config_c1', 'config_c2', 'c3_matrix_chunks', 'c3_events',
  'config_c3_twin', 'config_c3_first_rows', 'config_c4', 'config_c5',
]


def fixed_prob_csr(n_pre, n_post, prob, rng, sort=True):
  """Each row gets Binomial(n_post, prob) unique columns (the numpy twin of
  ``bp.conn.FixedProb(prob)(n_pre, n_post).require('pre2post')`` used by the
  reference tests, brainpylib/_src/event_ops/tests/test_event_csr_matvec.py:50)."""
  counts = np.empty(n_pre, dtype=np.int64)
  cols = []
  for r in range(n_pre):
    k = rng.binomial(n_post, prob)
    c = rng.choice(n_post, k, replace=False)
    cols.append(np.sort(c) if sort else c)
    counts[r] = k
  indices = np.concatenate(cols).astype(np.int32) if cols else np.zeros(0, np.int32)
  indptr = np.zeros(n_pre + 1, dtype=np.int32)
  np.cumsum(counts, out=indptr[1:])
  return indices, indptr


def fixed_degree_csr(n_pre, n_post, degree, rng):
  """``degree`` unique sorted columns per row."""
  indices = np.empty((n_pre, degree), dtype=np.int32)
  for r in range(n_pre):
    indices[r] = np.sort(rng.choice(n_post, degree, replace=False))
  indptr = np.arange(0, n_pre * degree + 1, degree, dtype=np.int32)
  return indices.reshape(-1), indptr


def config_c1():
  """event_csr_matvec, 4000 x 4000, p = 0.02, homogeneous 0.6, bool events 5 %, transpose."""
  r = np.random.default_rng(0)
  indices, indptr = fixed_prob_csr(4000, 4000, 0.02, r)
  data = np.array([0.6], dtype=np.float32)
  events = np.random.default_rng(1).random(4000) < 0.05
  return dict(data=data, indices=indices, indptr=indptr, events=events, shape=(4000, 4000), transpose=True)


def config_c2(n=100_000, degree=100):
  """csr_matvec, n x n, ``degree`` unique sorted columns per row, weights N(0,1), x ~ U(-1,1)."""
  r = np.random.default_rng(2)
  indices, indptr = fixed_degree_csr(n, n, degree, r)
  data = r.standard_normal(n * degree, dtype=np.float32)
  x = r.uniform(-1, 1, n).astype(np.float32)
  return dict(data=data, indices=indices, indptr=indptr, vector=x, shape=(n, n))


C3_ROWS_PER_CHUNK = 100_000
C3_DEGREE = 1000


def c3_matrix_chunks(n_neurons=1_000_000, rng=None):
  """Yields ``('indices', chunk_no, int32 array)`` for every chunk, then
  ``('data', chunk_no, float32 array)`` for every chunk, from ``default_rng(3)``.
  The chunking is part of the definition (the stream must not depend on host RAM).
  ``rng`` is returned to the caller through ``c3_events`` for the spike draws."""
  rng = np.random.default_rng(3) if rng is None else rng
  n_chunks = n_neurons // C3_ROWS_PER_CHUNK
  for c in range(n_chunks):
    yield 'indices', c, rng.integers(0, n_neurons, size=(C3_ROWS_PER_CHUNK, C3_DEGREE), dtype=np.int32).reshape(-1)
  for c in range(n_chunks):
    yield 'data', c, rng.random(C3_ROWS_PER_CHUNK * C3_DEGREE, dtype=np.float32)
  yield 'rng', -1, rng


def c3_events(rng, n_neurons=1_000_000, rate=0.01):
  """One step's spike vector (float32 0/1), drawn from the generator that produced the matrix."""
  return (rng.random(n_neurons) < rate).astype(np.float32)


def config_c3_twin(n_steps=4):
  """Reduced twin of C3 that a CPU can check: 1e5 neurons x 1000 synapses (1e8 nnz)."""
  n = 100_000
  out = {}
  for kind, c, arr in c3_matrix_chunks(n):
    if kind == 'rng':
      rng = arr
    else:
      out[kind] = arr
  events = [c3_events(rng, n) for _ in range(n_steps)]
  indptr = np.arange(0, n * C3_DEGREE + 1, C3_DEGREE, dtype=np.int32)
  return dict(data=out['data'], indices=out['indices'], indptr=indptr, events=events, shape=(n, n), transpose=True)


_c3_first_rows_cache = {}


def config_c3_first_rows(n_steps=2):
  """Pre-synaptic rows 0..99,999 (the first generation chunk: 1e8 synapses onto all 1e6 targets) of the FULL
  1e6-neuron matrix, with the spike vectors of the first ``n_steps`` steps.  ``events`` are the full vectors,
  ``events_masked`` the same with every spike outside rows 0..99,999 cleared: the product of the whole matrix
  with a masked vector equals the product of these rows with it, which a CPU can check."""
  if n_steps not in _c3_first_rows_cache:
    n = 1_000_000
    out = {}
    for kind, c, arr in c3_matrix_chunks(n):
      if kind == 'rng':
        rng = arr
      elif c == 0:
        out[kind] = arr
    events = [c3_events(rng, n) for _ in range(n_steps)]
    masked = []
    for e in events:
      m = np.zeros_like(e)
      m[:C3_ROWS_PER_CHUNK] = e[:C3_ROWS_PER_CHUNK]
      masked.append(m)
    indptr = np.arange(0, C3_ROWS_PER_CHUNK * C3_DEGREE + 1, C3_DEGREE, dtype=np.int32)
    _c3_first_rows_cache[n_steps] = dict(data=out['data'], indices=out['indices'], indptr=indptr, events=events,
                                         events_masked=masked, shape=(C3_ROWS_PER_CHUNK, n), transpose=True)
  return _c3_first_rows_cache[n_steps]


def config_c4(n=1_000_000):
  """jitconn event matvec, n x n, conn_prob 0.001, seed 42, bool events 2 %."""
  events = np.random.default_rng(4).random(n) < 0.02
  return dict(events=events, shape=(n, n), conn_prob=0.001, seed=42, transpose=False,
              uniform=dict(w_low=-0.1, w_high=0.1), homo=dict(weight=0.05), normal=dict(w_mu=0., w_sigma=0.01))


def config_c5(m=256, k=65536, n=65536):
  """jitconn matmat, X (m x k) ~ N(0,1) times a k x n just-in-time matrix, conn_prob 0.01, N(0, 0.01), seed 7."""
  X = np.random.default_rng(5).standard_normal((m, k), dtype=np.float32)
  return dict(matrix=X, shape=(k, n), conn_prob=0.01, w_mu=0., w_sigma=0.01, seed=7)
