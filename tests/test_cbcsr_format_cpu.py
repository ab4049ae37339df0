"""The column-blocked CSR format on the CPU: the conversion is plain tensor code, so its layout rules can be
checked without a GPU by rebuilding the dense matrix from the converted arrays."""
import numpy as np
import pytest
import torch

import cases
from brainpylib_b200 import event_ops


def _dense_from_blocked(cb):
  n_row, n_col = cb.shape
  dense = np.zeros((n_row, n_col), dtype=np.float64)
  offsets = cb.offsets.numpy().astype(np.int64)
  cols = cb.cols.numpy().view(np.uint16).astype(np.int64)      # stored as int16, read back unsigned
  data = cb.data.numpy()
  for r in range(n_row):
    for b in range(cb.n_blocks):
      for e in range(offsets[r, b], offsets[r, b + 1]):
        assert cols[e] < cb.block_width
        dense[r, b * cb.block_width + cols[e]] += data[e]
  return dense


@pytest.mark.parametrize('shape,block_width,rows_per_pass', [((40, 100), 32, 7), ((64, 70001 // 100), 256, 100_000),
                                                             ((30, 66000), 45056, 11), ((5, 7), None, 100_000)])
def test_conversion_keeps_every_synapse_in_its_row_and_block(shape, block_width, rows_per_pass):
  data, indices, indptr, _ = cases.csr_case(shape, 0.2 if shape[1] < 1000 else 0.002, 91)
  cb = event_ops.csr_to_column_blocked(torch.as_tensor(data), torch.as_tensor(indices), torch.as_tensor(indptr),
                                       shape=shape, block_width=block_width, rows_per_pass=rows_per_pass)
  assert cb.n_blocks == -(-shape[1] // cb.block_width)
  off = cb.offsets.numpy()
  assert np.array_equal(off[:, 0], indptr[:-1]) and np.array_equal(off[:, -1], indptr[1:])
  assert np.all(np.diff(off, axis=1) >= 0)
  want = np.zeros(shape, dtype=np.float64)
  for r in range(shape[0]):
    for e in range(indptr[r], indptr[r + 1]):
      want[r, indices[e]] += data[e]
  np.testing.assert_array_equal(_dense_from_blocked(cb), want)
  assert cb.nbytes() == 6 * data.shape[0] + 4 * (cb.n_blocks + 1) * shape[0]


def test_conversion_of_ragged_rows_with_duplicates_and_an_empty_matrix():
  lens = np.array([0, 1, 31, 32, 33, 700, 0, 5])
  data, indices, indptr, _ = cases.ragged_csr(lens, 300, 92)
  cb = event_ops.csr_to_column_blocked(torch.as_tensor(data), torch.as_tensor(indices), torch.as_tensor(indptr),
                                       shape=(lens.shape[0], 300), block_width=128)
  want = np.zeros((lens.shape[0], 300))
  for r in range(lens.shape[0]):
    for e in range(indptr[r], indptr[r + 1]):
      want[r, indices[e]] += data[e]
  np.testing.assert_allclose(_dense_from_blocked(cb), want, rtol=0, atol=1e-6)   # duplicates: order of float adds
  empty = event_ops.csr_to_column_blocked(torch.zeros(0), torch.zeros(0, dtype=torch.int32),
                                          torch.zeros(4, dtype=torch.int32), shape=(3, 9))
  assert empty.offsets.shape == (3, empty.n_blocks + 1) and int(empty.offsets.abs().sum()) == 0


def test_block_width_limits():
  with pytest.raises(ValueError):
    event_ops.csr_to_column_blocked(torch.zeros(0), torch.zeros(0, dtype=torch.int32),
                                    torch.zeros(4, dtype=torch.int32), shape=(3, 9), block_width=70000)
