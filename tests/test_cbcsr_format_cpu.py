"""The column-blocked matrix format without a GPU: the numpy statement of the layout (the one the GPU tests
hold the CUDA builder to, byte for byte) keeps every synapse in its row and block, and the Python side
refuses the block widths the kernel cannot take (odd widths would misalign its shared-memory arrays)."""
import numpy as np
import pytest
import torch

import cases
from brainpylib_b200 import event_ops
from brainpylib_b200.errors import GPUOperatorNotFound


def _dense(data, indices, indptr, shape, lo, hi):
  want = np.zeros((shape[0], hi - lo), dtype=np.float64)
  for r in range(shape[0]):
    for e in range(indptr[r], indptr[r + 1]):
      if lo <= indices[e] < hi:
        want[r, indices[e] - lo] += data[e]
  return want


@pytest.mark.parametrize('shape,block_width,col_range', [((40, 100), 32, None), ((64, 700), 256, None),
                                                         ((30, 66000), 32256, None), ((5, 7), 32, None),
                                                         ((50, 1000), 64, (250, 500)), ((50, 1000), 96, (990, 1000))])
def test_layout_model_keeps_every_synapse_in_its_row_and_block(shape, block_width, col_range):
  data, indices, indptr, _ = cases.csr_case(shape, 0.2 if shape[1] < 2000 else 0.002, 91)
  groups, offsets = cases.column_blocked_model(data, indices, indptr, shape[1], block_width, col_range)
  lo, hi = col_range or (0, shape[1])
  assert offsets.shape == (shape[0], max(1, -(-(hi - lo) // block_width)) + 1)
  assert groups.shape[0] == 48 * int(offsets[-1, -1]) and offsets[0, 0] == 0
  assert np.all(np.diff(offsets.astype(np.int64), axis=1) >= 0)
  assert np.array_equal(offsets[1:, 0], offsets[:-1, -1])          # rows lie back to back
  np.testing.assert_array_equal(cases.dense_from_column_blocked(groups, offsets, hi - lo, block_width),
                                _dense(data, indices, indptr, shape, lo, hi))


def test_layout_model_ragged_rows_duplicates_and_padding():
  lens = np.array([0, 1, 7, 8, 9, 31, 32, 33, 700, 0, 5])
  data, indices, indptr, _ = cases.ragged_csr(lens, 300, 92)
  groups, offsets = cases.column_blocked_model(data, indices, indptr, 300, 128)
  np.testing.assert_allclose(cases.dense_from_column_blocked(groups, offsets, 300, 128),
                             _dense(data, indices, indptr, (lens.shape[0], 300), 0, 300), rtol=0, atol=1e-6)
  # a segment of k synapses takes ceil(k / 8) records: row 1 (one synapse) takes exactly one
  assert int(offsets[1, -1] - offsets[1, 0]) == 1
  assert int(offsets[0, -1] - offsets[0, 0]) == 0


@pytest.mark.parametrize('width', [0, 31, 33, 1000 + 1, 32256 + 32, 70000])
def test_block_widths_the_kernel_cannot_take_are_refused(width):
  with pytest.raises(ValueError):
    event_ops.check_block_width(width)


def test_default_block_width_is_a_multiple_of_32_within_the_limit():
  for n_col in (1, 7, 4000, 125_000, 1_000_000, 50_000_000):
    w = event_ops.default_block_width(n_col)
    event_ops.check_block_width(w)


def test_the_builder_has_no_cpu_path():
  with pytest.raises(GPUOperatorNotFound):
    event_ops.csr_to_column_blocked(torch.zeros(0), torch.zeros(0, dtype=torch.int32),
                                    torch.zeros(4, dtype=torch.int32), shape=(3, 9))
