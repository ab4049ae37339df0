"""GPU checks of event_info (spike compaction): count == sum(events) for the lengths the reference
tests use (brainpylib/_src/event_ops/tests/test_event_info_collection.py:19-59), and — what the
reference never checks — the indices themselves: ascending, equal to numpy's nonzero, padded with -1."""
import numpy as np
import pytest
import torch

import brainpylib_b200 as bpl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('dtype', [np.bool_, np.int32, np.int64, np.float32, np.float64])
def test_event_info_matches_numpy(cuda, dtype):
  rng = np.random.default_rng(0)
  for n in (1, 2, 31, 32, 33, 100, 4095, 4096, 4097, 10000, 100000, 1000001):
    for rate in (0.0, 0.1, 1.0):
      ev = (rng.random(n) < rate)
      vals = ev.astype(dtype) if dtype == np.bool_ else (ev * rng.integers(1, 5, n)).astype(dtype)
      ids, num = bpl.event_info(torch.as_tensor(vals).to(cuda))
      want = np.nonzero(vals)[0]
      assert int(num) == want.shape[0] == int(ev.sum())
      ids = ids.cpu().numpy()
      assert ids.dtype == np.int32 and ids.shape == (n,)
      np.testing.assert_array_equal(ids[:want.shape[0]], want)
      assert (ids[want.shape[0]:] == -1).all()


def test_event_info_batch_and_errors(cuda):
  rng = np.random.default_rng(1)
  ev = rng.random((7, 5000)) < 0.2
  ids, num = bpl.event_info(torch.as_tensor(ev).to(cuda))
  assert ids.shape == (7, 5000) and num.shape == (7,)
  for r in range(7):
    want = np.nonzero(ev[r])[0]
    assert int(num[r]) == want.shape[0]
    np.testing.assert_array_equal(ids[r, :want.shape[0]].cpu().numpy(), want)
    assert (ids[r, want.shape[0]:] == -1).all()
  with pytest.raises(TypeError):
    bpl.event_info(torch.zeros(2, 2, 2, dtype=torch.bool, device=cuda))
  # the compacted list drives the transposed event product: same active rows as the operator sees
  y1, n1 = bpl.event_info(torch.as_tensor(ev[0]).to(cuda))
  assert int(n1) == int(ev[0].sum())
