"""Single-GPU checks of the spike-exchange kernels (world = 1: the rank pushes to itself): slot
addressing, the arrival counters across repeated use of a slot, and the bounded wait, which must
give up with a status instead of spinning when nothing arrives.  Push and wait are separate launches
on one stream here, so neither ever waits on a kernel that is not already complete or absent."""
import numpy as np
import pytest
import torch

from brainpylib_b200 import sharded

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('dtype', [torch.float32, torch.bool, torch.uint8])
def test_push_then_wait_roundtrip(cuda, dtype):
  n = 300_000 + 16          # several CTAs per destination
  ex = sharded.PushExchange(n, dtype=dtype, device=cuda, slots=4, max_polls=1000)
  g = torch.Generator(device='cpu').manual_seed(0)
  for step in range(11):                      # every slot is reused several times
    slot = step % ex.slots
    ev = (torch.rand(n, generator=g) < 0.3)
    ev = ev.to(dtype) if dtype != torch.float32 else ev.float() * 1.5
    ev = ev.to(cuda)
    ex.push(ev, slot)
    ex.wait(slot)
    assert torch.equal(ex.events(slot), ev)
  ex.check()


def test_wait_without_push_times_out_and_returns(cuda):
  ex = sharded.PushExchange(1024, dtype=torch.float32, device=cuda, slots=4, max_polls=200)
  ex.wait(2)                                   # nothing was pushed into slot 2: the wait must run out
  torch.cuda.synchronize()                     # ... and the kernel must have returned
  assert ex.timed_out()
  with pytest.raises(RuntimeError, match='ran out of polls'):
    ex.check()
  # the device is still usable afterwards
  assert torch.ones(8, device=cuda).sum().item() == 8


def test_exchange_argument_checks(cuda):
  ex = sharded.PushExchange(1024, dtype=torch.float32, device=cuda)
  with pytest.raises(ValueError):
    ex.push(torch.zeros(10, device=cuda), 0)
  with pytest.raises(RuntimeError):
    ex.wait(9)                                 # slot out of range -> status from the C ABI
  with pytest.raises(RuntimeError):
    ex.push(torch.zeros(1024, device=cuda), 7)


@pytest.mark.parametrize('dtype', [torch.float32, torch.bool])
def test_compacted_push_feeds_the_scatter_directly(cuda, dtype):
  """world = 1: the fused compaction + push assembles the spike list, the wait zero-fills y, and the
  list-driven scatter gives what event_csr_matvec gives on the same spikes (same kernel, same list)."""
  import cases
  import brainpylib_b200 as bpl
  shape = (9000, 3000)
  data, indices, indptr, rng = cases.csr_case(shape, 0.01, 17)
  d, ix, ptr = (torch.as_tensor(a).to(cuda) for a in (data, indices, indptr))
  ex = sharded.PushExchange(shape[0], dtype=torch.float32, device=cuda, slots=4, max_polls=1000)
  y = torch.full((shape[1],), float('nan'), device=cuda)
  for step in range(6):
    slot = step % 4
    ev = torch.as_tensor(rng.random(shape[0]) < (0.3 if step % 2 else 0.01)).to(cuda)
    ev = ev if dtype == torch.bool else ev.float() * 2.0
    ex.push_compacted(ev, slot)
    ex.wait_zero(slot, y)
    ex.scatter_from_list(d, ix, ptr, slot, y, shape[1])
    want = bpl.event_csr_matvec(d, ix, ptr, ev, shape=shape, transpose=True)
    torch.testing.assert_close(y, want, rtol=1e-5, atol=1e-4)
    counts = ex.spike_list(slot)[: ex.n_chunks]
    assert int(counts.sum()) == int((ev != 0).sum())
  ex.check()


@pytest.mark.parametrize('dtype,shape,density', [(torch.float32, (9000, 3000), 0.01), (torch.bool, (9000, 3000), 0.01),
                                                 # 49 chunks of events: more than the kernel's pushing blocks (1/16 of
                                                 # the grid), so each of them compacts and pushes several chunks
                                                 (torch.float32, (200000, 3000), 0.002)])
def test_fused_step_kernel_matches_the_operator(cuda, dtype, shape, density):
  """world = 1: prime + one launch per step (push of step t+1, zero-fill of the other output buffer, bounded
  wait, scatter of step t) gives, step after step and across slot reuse, what event_csr_matvec gives."""
  import cases
  import brainpylib_b200 as bpl
  data, indices, indptr, rng = cases.csr_case(shape, density, 23)
  d, ix, ptr = (torch.as_tensor(a).to(cuda) for a in (data, indices, indptr))
  ex = sharded.PushExchange(shape[0], dtype=torch.float32, device=cuda, slots=4, max_polls=1000)
  steps = 7
  evs = []
  for s in range(steps):
    ev = torch.as_tensor(rng.random(shape[0]) < (0.3 if s % 2 else 0.01)).to(cuda)
    evs.append(ev if dtype == torch.bool else ev.float() * 2.0)
  y = [torch.full((shape[1],), float('nan'), device=cuda) for _ in range(2)]
  ex.prime(evs[0], y[0])
  for s in range(steps):
    nxt = evs[s + 1] if s + 1 < steps else None
    ex.step(d, ix, ptr, y[s % 2], y[(s + 1) % 2] if nxt is not None else None, nxt)
    want = bpl.event_csr_matvec(d, ix, ptr, evs[s], shape=shape, transpose=True)
    torch.testing.assert_close(y[s % 2], want, rtol=1e-5, atol=1e-4)
  ex.check()
  # a second run on the same object starts where the counter stands
  ex.prime(evs[3], y[1])
  ex.step(d, ix, ptr, y[1], None, None)
  torch.testing.assert_close(y[1], bpl.event_csr_matvec(d, ix, ptr, evs[3], shape=shape, transpose=True),
                             rtol=1e-5, atol=1e-4)
  ex.check()


def test_fused_step_times_out_without_a_prime(cuda):
  """A step whose lists never arrive gives up after max_polls, reports it, leaves y untouched and the GPU usable."""
  import cases
  shape = (5000, 2000)
  data, indices, indptr, rng = cases.csr_case(shape, 0.01, 5)
  d, ix, ptr = (torch.as_tensor(a).to(cuda) for a in (data, indices, indptr))
  ex = sharded.PushExchange(shape[0], dtype=torch.float32, device=cuda, slots=4, max_polls=50)
  y = torch.zeros(shape[1], device=cuda)
  ex.step(d, ix, ptr, y, None, None)
  torch.cuda.synchronize()
  with pytest.raises(Exception):
    ex.check()
  assert float(y.abs().sum()) == 0.0


@pytest.mark.parametrize('dtype,shape,density,accumulate,width',
                         [(torch.float32, (9000, 3000), 0.01, 'float', 1024), (torch.bool, (9000, 3000), 0.01, 'fixed', 512),
                          # 49 chunks of events over 16 exchanging teams: each pushes several chunks in turn
                          (torch.float32, (200000, 3000), 0.002, 'float', None),
                          (torch.bool, (70000, 40000), 0.003, 'fixed', 20416)])
def test_fused_step_on_a_prepared_shard_matches_the_operator(cuda, dtype, shape, density, accumulate, width):
  """world = 1: the one-launch step on the column-blocked layout (exchange blocks beside the scatter's (block, share)
  CTAs) gives, step after step and across slot reuse, what the stand-alone prepared operator gives: within float32
  summation order, and with fixed-point accumulation within the rounding of adding the few CTA shares of a block
  (the two launches split the rows over a different number of CTAs)."""
  import cases
  import brainpylib_b200 as bpl
  data, indices, indptr, rng = cases.csr_case(shape, density, 29)
  d, ix, ptr = (torch.as_tensor(a).to(cuda) for a in (data, indices, indptr))
  prepared = bpl.csr_to_column_blocked(d, ix, ptr, shape=shape, block_width=width, accumulate=accumulate)
  ex = sharded.PushExchange(shape[0], dtype=torch.float32, device=cuda, slots=4, max_polls=1000)
  steps = 6
  evs = []
  for s in range(steps):
    ev = torch.as_tensor(rng.random(shape[0]) < (0.3 if s % 2 else 0.01)).to(cuda)
    evs.append(ev if dtype == torch.bool else ev.float() * 2.0)
  y = [torch.full((shape[1],), float('nan'), device=cuda) for _ in range(2)]
  ex.prime(evs[0], y[0])
  launches = [ex.step_prepared_call(prepared, y[s % 2], y[(s + 1) % 2] if s + 1 < steps else None,
                                    evs[s + 1] if s + 1 < steps else None, torch.cuda.current_stream().cuda_stream)
              for s in range(steps)]
  for s in range(steps):
    if s % 2:
      launches[s]()
    else:
      ex.step_prepared(prepared, y[s % 2], y[(s + 1) % 2] if s + 1 < steps else None, evs[s + 1] if s + 1 < steps else None)
    want = bpl.event_csr_matvec(d, ix, ptr, evs[s], shape=shape, transpose=True, prepared=prepared)
    if accumulate == 'fixed':
      torch.testing.assert_close(y[s % 2], want, rtol=1e-6, atol=1e-5)
    else:
      torch.testing.assert_close(y[s % 2], want, rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(want, bpl.event_csr_matvec(d, ix, ptr, evs[s], shape=shape, transpose=True),
                               rtol=1e-4, atol=1e-3)
  ex.check()


def test_prepared_step_refuses_a_shard_of_another_shape(cuda):
  import cases
  import brainpylib_b200 as bpl
  data, indices, indptr, _ = cases.csr_case((3000, 2000), 0.01, 3)
  d, ix, ptr = (torch.as_tensor(a).to(cuda) for a in (data, indices, indptr))
  prepared = bpl.csr_to_column_blocked(d, ix, ptr, shape=(3000, 2000), block_width=1024)
  ex = sharded.PushExchange(4000, dtype=torch.float32, device=cuda, slots=4, max_polls=50)
  with pytest.raises(ValueError, match='rows'):
    ex.step_prepared(prepared, torch.zeros(2000, device=cuda), None, None)
  ex = sharded.PushExchange(3000, dtype=torch.float32, device=cuda, slots=4, max_polls=50)
  with pytest.raises(ValueError, match='entries of the shard'):
    ex.step_prepared(prepared, torch.zeros(1999, device=cuda), None, None)
