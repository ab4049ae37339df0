"""GPU parity of the legacy scatter operators against the CPU oracle and the golden outputs
of the reference's CPU kernels (lib/cpu_atomic_sum.cc, lib/cpu_atomic_prod.cc)."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden'))
import cases  # noqa: E402
import make_golden  # noqa: E402
import brainpylib_b200 as bpl  # noqa: E402
from oracle import cpu  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'stored_matrix.npz'))
GOLD = [c for c in make_golden.golden_cases() if c[1] == 'coo_atomic']


@pytest.mark.parametrize('name,kind,kw', GOLD, ids=[c[0] for c in GOLD])
@pytest.mark.parametrize('itype', [torch.int32, torch.int64])
def test_coo_atomic_matches_reference_golden(cuda, name, kind, kw, itype):
  inp = make_golden.build_inputs(kind, kw)
  fn = bpl.coo_atomic_sum if inp['op'] == 'sum' else bpl.coo_atomic_prod
  values = torch.as_tensor(inp['values']).to(cuda)
  post = torch.as_tensor(inp['post']).to(cuda).to(itype)
  pre = None if inp['homo'] else torch.as_tensor(inp['pre']).to(cuda).to(itype)
  y = fn(values, post, inp['post_num'], pre).cpu().numpy()
  np.testing.assert_allclose(y, GOLDEN[name], rtol=2e-5, atol=1e-4)


@pytest.mark.parametrize('dtype', [np.float32, np.float64])
@pytest.mark.parametrize('homo', [True, False])
def test_csr_and_coo_event_sum(cuda, dtype, homo):
  shape = (500, 400)
  data, indices, indptr, rng = cases.csr_case(shape, 0.1, 71, homo=0.6 if homo else None, dtype=dtype)
  events = rng.random(shape[0]) < 0.2
  t = lambda a: torch.as_tensor(a).to(cuda)
  want = cpu.event_csr_matvec(data, indices, indptr, events, shape=shape, transpose=True)
  y = bpl.csr_event_sum(t(events), (t(indices), t(indptr)), shape[1], t(data))
  if homo:
    assert y.cpu().numpy().tobytes() == want.tobytes()
  else:
    np.testing.assert_allclose(y.cpu().numpy().astype(dtype), want, rtol=1e-5, atol=1e-3)
  row = np.repeat(np.arange(shape[0], dtype=np.int32), np.diff(indptr))
  want2 = cpu.coo_event_sum(events, row, indices, shape[1], data)
  y2 = bpl.coo_event_sum(t(events), t(row), t(indices), shape[1], t(data))
  np.testing.assert_allclose(y2.cpu().numpy(), want2, rtol=1e-5, atol=1e-3)
  np.testing.assert_allclose(want2, want, rtol=1e-5, atol=1e-3)


def test_legacy_csr_event_sum_target(cuda):
  """The `gpu_csr_event_sum_*` custom-call targets themselves (no workspace, i32 and i64 indices)."""
  from brainpylib_b200 import _lib, gpu_ops
  shape = (300, 200)
  data, indices, indptr, rng = cases.csr_case(shape, 0.2, 72)
  events = rng.random(shape[0]) < 0.3
  want = cpu.event_csr_matvec(data, indices, indptr, events, shape=shape, transpose=True)
  for itype, suffix in ((torch.int32, 'i32'), (torch.int64, 'i64')):
    bufs = [torch.as_tensor(events).to(cuda), torch.as_tensor(indices).to(cuda).to(itype),
            torch.as_tensor(indptr).to(cuda).to(itype), torch.as_tensor(data).to(cuda),
            torch.empty(shape[1], device=cuda)]
    _lib.call(f'gpu_csr_event_sum_heter_f32_{suffix}', bufs, gpu_ops.build_csr_event_sum_descriptor(*shape))
    np.testing.assert_allclose(bufs[-1].cpu().numpy(), want, rtol=1e-5, atol=1e-3)
