"""Seeded inputs shared by the parity tests (numpy only)."""
import numpy as np

from brainpylib_b200.workloads import fixed_prob_csr

# shapes of the reference's own tests
EVENT_CSR_SHAPES = [(100, 200), (200, 200), (200, 100), (10, 1000), (2, 10000), (1000, 10), (10000, 2)]
# brainpylib/_src/event_ops/tests/test_event_csr_matvec.py:37-43
CSR_SHAPES = [(100, 200), (200, 100), (10, 1000), (2, 2000)]
# brainpylib/_src/sparse_ops/tests/test_sparse_csr_matvec.py:48-50,78-82
JITCONN_SHAPES = [(100, 200), (10, 1000), (2, 1000), (1000, 10), (1000, 2)]
# brainpylib/_src/jitconn_ops/tests/test_event_matvec.py:10-14
MATMAT_SHAPES = JITCONN_SHAPES + [(200, 200)]
# brainpylib/_src/jitconn_ops/tests/matmat_testcase.py:10-15


def csr_case(shape, prob, seed, *, homo=None, dtype=np.float32, sort=True):
  rng = np.random.default_rng(seed)
  indices, indptr = fixed_prob_csr(shape[0], shape[1], prob, rng, sort=sort)
  if homo is None:
    data = rng.standard_normal(indices.shape[0]).astype(dtype)
  else:
    data = np.array([homo], dtype=dtype)
  return data, indices, indptr, rng


def ragged_csr(row_lengths, n_col, seed, dtype=np.float32, duplicates=True):
  """Rows of prescribed lengths (0, 1, 31, 32, 33, 1000 ...), unsorted, duplicates allowed."""
  rng = np.random.default_rng(seed)
  lens = np.asarray(row_lengths, dtype=np.int64)
  indptr = np.zeros(lens.shape[0] + 1, dtype=np.int32)
  np.cumsum(lens, out=indptr[1:])
  indices = rng.integers(0, n_col, size=int(lens.sum()), dtype=np.int32)
  data = rng.standard_normal(indices.shape[0]).astype(dtype)
  return data, indices, indptr, rng


def events_like(rng, n, rate, dtype):
  ev = rng.random(n) < rate
  if dtype == np.bool_:
    return ev
  return ev.astype(dtype)
