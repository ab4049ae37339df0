"""Runs over spike trains in pinned host memory (bpl_run_host_steps / bpl_sharded_run_host_steps): every step's
result must be what the operator gives for that step's spikes on the device, for rings that wrap many times."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture
def cuda():
  if not torch.cuda.is_available():
    pytest.skip('needs a CUDA device')
  return torch.device('cuda', 0)


def _case(shape, density, seed, cuda):
  import cases
  data, indices, indptr, rng = cases.csr_case(shape, density, seed)
  return tuple(torch.as_tensor(a).to(cuda) for a in (data, indices, indptr)), rng


@pytest.mark.parametrize('layout,group', [('csr', 4), ('prepared', 4), ('prepared_fixed', 1), ('homo', 16), ('csr', 3)])
@pytest.mark.parametrize('dtype', [torch.float32, torch.bool])
def test_host_steps_match_the_operator_step_by_step(cuda, layout, group, dtype):
  import brainpylib_b200 as bpl
  shape = (20000, 7000)
  (d, ix, ptr), rng = _case(shape, 0.004, 41, cuda)
  if layout == 'homo':
    d = torch.tensor([0.75], device=cuda)
  steps = 11
  ev = torch.from_numpy(rng.random((steps, shape[0])) < 0.02)
  ev = (ev if dtype == torch.bool else ev.float() * 1.5).pin_memory()
  out = torch.full((steps, shape[1]), float('nan')).pin_memory()
  prepared = None
  if layout.startswith('prepared'):
    prepared = bpl.csr_to_column_blocked(d, ix, ptr, shape=shape, block_width=2048,
                                         accumulate='fixed' if layout.endswith('fixed') else 'float')
  runner = bpl.HostSteps(prepared if prepared is not None else (d, ix, ptr), shape=shape, events_dtype=dtype,
                         group=group)
  ms = runner.run(ev, out)
  assert ms > 0
  for s in range(steps):
    want = bpl.event_csr_matvec(d, ix, ptr, ev[s].to(cuda), shape=shape, transpose=True, prepared=prepared)
    torch.testing.assert_close(out[s].to(cuda), want, rtol=1e-5, atol=1e-5)
  # fewer result slots than steps: the last `slots` steps remain; a second run reuses the rings
  few = torch.zeros((2, shape[1])).pin_memory()
  runner.run(ev, few)
  for s in (steps - 2, steps - 1):
    torch.testing.assert_close(few[s % 2], out[s], rtol=1e-5, atol=1e-5)


def test_host_steps_refuse_pageable_memory_and_wrong_shapes(cuda):
  import brainpylib_b200 as bpl
  shape = (3000, 2000)
  (d, ix, ptr), _ = _case(shape, 0.01, 5, cuda)
  runner = bpl.HostSteps((d, ix, ptr), shape=shape)
  good_ev, good_out = torch.zeros((2, 3000)).pin_memory(), torch.zeros((2, 2000)).pin_memory()
  with pytest.raises(ValueError, match='pinned'):
    runner.run(torch.zeros((2, 3000)), good_out)
  with pytest.raises(ValueError, match='host_events must be'):
    runner.run(torch.zeros((2, 2999)).pin_memory(), good_out)
  with pytest.raises(ValueError, match='host_out must be'):
    runner.run(good_ev, torch.zeros((2, 2001)).pin_memory())
  runner.run(good_ev, good_out)
  assert float(good_out.abs().sum()) == 0.0


@pytest.mark.parametrize('dtype,accumulate,group', [(torch.float32, 'float', 4), (torch.bool, 'fixed', 1),
                                                    (torch.float32, 'fixed', 5), (torch.bool, 'float', 16)])
def test_sharded_host_steps_on_one_rank(cuda, dtype, accumulate, group):
  """world = 1: prime, one launch per step and the three-stream pipeline, against the operator step by step."""
  import brainpylib_b200 as bpl
  from brainpylib_b200 import sharded
  shape = (50000, 9000)
  (d, ix, ptr), rng = _case(shape, 0.003, 43, cuda)
  prepared = bpl.csr_to_column_blocked(d, ix, ptr, shape=shape, block_width=4096, accumulate=accumulate)
  ex = sharded.PushExchange(shape[0], dtype=torch.float32, device=cuda, slots=4, max_polls=100000)
  steps = 13
  ev = torch.from_numpy(rng.random((steps, shape[0])) < 0.02)
  ev = (ev if dtype == torch.bool else ev.float()).pin_memory()
  out = torch.full((steps, shape[1]), float('nan')).pin_memory()
  for _ in range(2):            # a second run continues on the same exchange object
    ms = ex.run_host_steps(prepared, ev, out, group=group)
    ex.check()
    assert ms > 0
    for s in range(steps):
      want = bpl.event_csr_matvec(d, ix, ptr, ev[s].to(cuda), shape=shape, transpose=True, prepared=prepared)
      torch.testing.assert_close(out[s].to(cuda), want, rtol=1e-5, atol=1e-5)
    out.fill_(float('nan'))


@pytest.mark.parametrize('steps', [1, 2, 3, 4, 7])
def test_runs_shorter_than_a_group_and_ragged_last_groups(cuda, steps):
  """Runs of fewer steps than one group, exactly one group, and a ragged last group, single-device and sharded."""
  import brainpylib_b200 as bpl
  from brainpylib_b200 import sharded
  shape = (12000, 5000)
  (d, ix, ptr), rng = _case(shape, 0.004, 47, cuda)
  prepared = bpl.csr_to_column_blocked(d, ix, ptr, shape=shape, block_width=1024)
  ev = torch.from_numpy(rng.random((steps, shape[0])) < 0.03).float().pin_memory()
  want = [bpl.event_csr_matvec(d, ix, ptr, ev[s].to(cuda), shape=shape, transpose=True, prepared=prepared)
          for s in range(steps)]
  out = torch.full((steps, shape[1]), float('nan')).pin_memory()
  bpl.HostSteps(prepared, shape=shape, group=3).run(ev, out)
  for s in range(steps):
    torch.testing.assert_close(out[s].to(cuda), want[s], rtol=1e-5, atol=1e-5)
  ex = sharded.PushExchange(shape[0], dtype=torch.float32, device=cuda, slots=4, max_polls=100000)
  for shard in (prepared, (d, ix, ptr)):              # the rank's shard in either storage
    out.fill_(float('nan'))
    ex.run_host_steps(shard, ev, out, group=3)
    ex.check()
    for s in range(steps):
      torch.testing.assert_close(out[s].to(cuda), want[s], rtol=1e-5, atol=1e-5)
  assert sharded.preferred_layout(500_000) == 'prepared' and sharded.preferred_layout(125_000) == 'csr'
