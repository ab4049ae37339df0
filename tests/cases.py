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


def column_blocked_model(data, indices, indptr, n_col, block_width, col_range=None):
  """Numpy statement of the column-blocked layout the GPU builder must produce, byte for byte:
  per (row, block) segment whole records of 8 synapses (float32 w[8], uint16 c[8]), CSR order kept
  inside a segment, zero padding; offsets[r, b] in records.  Returns (groups uint8, offsets uint32)."""
  lo, hi = (0, n_col) if col_range is None else col_range
  n_row = indptr.shape[0] - 1
  n_blocks = max(1, -(-(hi - lo) // block_width))
  offsets = np.zeros((n_row, n_blocks + 1), dtype=np.uint32)
  records = []
  run = 0
  for r in range(n_row):
    seg = slice(indptr[r], indptr[r + 1])
    c, w = indices[seg].astype(np.int64), (np.broadcast_to(data, indices.shape)[seg] if data.shape[0] == 1 else data[seg])
    keep = (c >= lo) & (c < hi)
    c, w = c[keep] - lo, w[keep]
    blk = c // block_width
    for b in range(n_blocks):
      offsets[r, b] = run
      m = blk == b
      k = int(m.sum())
      n_rec = -(-k // 8)
      ws = np.zeros(n_rec * 8, dtype=np.float32)
      cs = np.zeros(n_rec * 8, dtype=np.uint16)
      ws[:k], cs[:k] = w[m], (c[m] - b * block_width).astype(np.uint16)
      for g in range(n_rec):
        records.append(ws[8 * g:8 * g + 8].tobytes() + cs[8 * g:8 * g + 8].tobytes())
      run += n_rec
    offsets[r, n_blocks] = run
  groups = np.frombuffer(b''.join(records), dtype=np.uint8) if records else np.zeros(0, np.uint8)
  return groups, offsets


def dense_from_column_blocked(groups, offsets, n_col_kept, block_width):
  """Dense float64 matrix (rows x kept columns) rebuilt from the column-blocked arrays."""
  n_row, n_blocks = offsets.shape[0], offsets.shape[1] - 1
  dense = np.zeros((n_row, n_col_kept), dtype=np.float64)
  rec = groups.reshape(-1, 48)
  for r in range(n_row):
    for b in range(n_blocks):
      for g in range(int(offsets[r, b]), int(offsets[r, b + 1])):
        w = rec[g, :32].copy().view(np.float32)
        c = rec[g, 32:].copy().view(np.uint16).astype(np.int64)
        for k in range(8):
          if w[k] != 0:
            assert c[k] < block_width
            dense[r, b * block_width + c[k]] += w[k]
  return dense
