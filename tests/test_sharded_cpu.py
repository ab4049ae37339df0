"""World-size-2 checks of the multi-GPU sharding logic on CPU ranks (gloo): the column shards
tile the matrix exactly, and all-gather + local product on each shard reproduces the oracle's
result for the whole matrix.  The local product is the CPU oracle here (the CUDA operator is
exercised by the GPU tests); what is under test is the partition and the exchange."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from brainpylib_b200 import sharded
from oracle import cpu


def _free_port():
  with socket.socket() as s:
    s.bind(('127.0.0.1', 0))
    return s.getsockname()[1]


def _oracle_op(data, indices, indptr, events, *, shape, transpose):
  y = cpu.event_csr_matvec(data.numpy(), indices.numpy(), indptr.numpy(), events.numpy(), shape=shape,
                           transpose=transpose)
  return torch.from_numpy(y)


def _case(homo=False):
  n_pre, n_post = 600, 501          # n_post not divisible by the world size: ragged last range
  data, indices, indptr, rng = cases.csr_case((n_pre, n_post), 0.05, 5, homo=0.6 if homo else None)
  events = [(rng.random(n_pre) < r) for r in (0.1, 0.0, 1.0)]
  return n_pre, n_post, data, indices, indptr, events


def test_column_shards_tile_the_matrix():
  n_pre, n_post, data, indices, indptr, _ = _case()
  t = [torch.from_numpy(a) for a in (data, indices, indptr)]
  for world in (1, 2, 3, 8):
    seen = 0
    dense = np.zeros((n_pre, n_post), dtype=np.float64)
    for rank in range(world):
      d, idx, ptr, (lo, hi) = sharded.shard_csr_by_columns(t[0], t[1], t[2], n_post, rank, world)
      assert ptr[0] == 0 and ptr[-1] == idx.shape[0] == d.shape[0]
      assert idx.numel() == 0 or (0 <= idx.min() and idx.max() < hi - lo)
      seen += idx.shape[0]
      rows = np.repeat(np.arange(n_pre), np.diff(ptr.numpy()))
      np.add.at(dense, (rows, idx.numpy() + lo), d.numpy())
    assert seen == indices.shape[0]
    want = np.zeros_like(dense)
    np.add.at(want, (np.repeat(np.arange(n_pre), np.diff(indptr)), indices), data)
    np.testing.assert_array_equal(dense, want)
  assert sharded.column_range(10, 3, 4) == (9, 10) and sharded.column_range(10, 0, 1) == (0, 10)


def _worker(rank, world, port, homo, out_queue):
  os.environ['MASTER_ADDR'] = '127.0.0.1'
  os.environ['MASTER_PORT'] = str(port)
  dist.init_process_group('gloo', rank=rank, world_size=world)
  try:
    n_pre, n_post, data, indices, indptr, events = _case(homo)
    t = [torch.from_numpy(a) for a in (data, indices, indptr)]
    d, idx, ptr, rng_cols = sharded.shard_csr_by_columns(t[0], t[1], t[2], n_post, rank, world)
    op = sharded.ShardedEventCSR(d, idx, ptr, n_pre, rng_cols, local_op=_oracle_op)
    lo_s, hi_s = op.source_range()
    results = []
    for ev in events:
      for dtype in (np.bool_, np.float32):
        local = torch.from_numpy(ev[lo_s:hi_s].astype(dtype))
        results.append(op.step(local).numpy())
    out_queue.put((rank, rng_cols, results))
  finally:
    dist.destroy_process_group()


def _run_world(world, homo):
  ctx = mp.get_context('spawn')
  q = ctx.Queue()
  port = _free_port()
  procs = [ctx.Process(target=_worker, args=(r, world, port, homo, q)) for r in range(world)]
  for p in procs:
    p.start()
  got = [q.get(timeout=120) for _ in range(world)]
  for p in procs:
    p.join(timeout=60)
    assert p.exitcode == 0
  return sorted(got)


def test_two_ranks_reproduce_the_single_device_result():
  for homo in (False, True):
    n_pre, n_post, data, indices, indptr, events = _case(homo)
    got = _run_world(2, homo)
    k = 0
    for ev in events:
      for dtype in (np.bool_, np.float32):
        want = cpu.event_csr_matvec(data, indices, indptr, ev.astype(dtype), shape=(n_pre, n_post), transpose=True)
        y = np.concatenate([res[k] for _, _, res in got])
        assert y.shape == want.shape
        # same per-target addition order inside a shard as in the whole matrix: bit-exact
        assert y.tobytes() == want.tobytes()
        k += 1
    assert [r for _, r, _ in got] == [(0, 251), (251, 501)]


# ------------------------------------------------------------------------------------------
# The one-launch-per-step protocol (sharded_step_kernel) as a host-side model: every rank runs its launches
# in order; launch t first stores its spikes of step t + 1 into slot (t + 1) % slots of EVERY rank, then may
# only finish once the lists of step t from every rank have arrived in its own slot t % slots (generation
# t // slots + 1), reads them, and publishes the arrival of step t + 1.  A random scheduler interleaves the
# ranks; the model checks that a rank never reads a list that belongs to another step (overwritten early or
# not yet written) and that nobody deadlocks.
# ------------------------------------------------------------------------------------------
def _simulate_step_protocol(world, slots, steps, seed):
  import random
  rng = random.Random(seed)
  content = [[[None] * world for _ in range(slots)] for _ in range(world)]   # [rank][slot][src] = step stored
  flags = [[[0] * world for _ in range(slots)] for _ in range(world)]        # [rank][slot][src] = arrivals
  # launch t on a rank: first the stores of step t + 1 everywhere; then, in EITHER order (pushing blocks do not
  # wait for scattering blocks), the publication of step t + 1 and the bounded wait + read of step t.
  t_of = [0] * world
  stored = [False] * world
  read = [False] * world
  published = [False] * world
  for r in range(world):                               # prime: every rank stores and publishes step 0
    for q in range(world):
      content[q][0][r] = 0
      flags[q][0][r] += 1
  violations, idle = [], 0
  while min(t_of) < steps and idle < 10000:
    r = rng.randrange(world)
    t = t_of[r]
    if t >= steps:
      idle += 1
      continue
    progressed = True
    if not stored[r]:
      for q in range(world):
        content[q][(t + 1) % slots][r] = t + 1        # peer stores of the next step's list
      stored[r] = True
    elif not published[r] and (read[r] or rng.random() < 0.5):
      for q in range(world):
        flags[q][(t + 1) % slots][r] += 1             # arrival of step t + 1 published
      published[r] = True
    elif not read[r]:
      slot, expected = t % slots, t // slots + 1
      if all(flags[r][slot][src] >= expected for src in range(world)):
        for src in range(world):
          if content[r][slot][src] != t:
            violations.append((r, t, src, content[r][slot][src]))
        read[r] = True
      else:
        progressed = False
    if read[r] and published[r]:
      t_of[r] = t + 1
      stored[r] = read[r] = published[r] = False
    idle = 0 if progressed else idle + 1
  return violations, min(t_of) >= steps


def test_step_protocol_is_safe_with_four_slots_and_live():
  for world in (2, 3, 8):
    for seed in range(20):
      violations, finished = _simulate_step_protocol(world, slots=4, steps=40, seed=seed)
      assert finished, 'the protocol deadlocked'
      assert not violations, violations[:3]


def test_step_protocol_model_detects_too_few_slots():
  """The model has teeth: with three slots some interleaving lets a fast rank overwrite a list a slow one
  has not read yet (the C entry point refuses slots < 4)."""
  found = False
  for seed in range(200):
    violations, _ = _simulate_step_protocol(2, slots=3, steps=40, seed=seed)
    found = found or bool(violations)
  assert found


def test_matmat_column_shard_calls_the_operator_with_offset_seed(monkeypatch):
  """Host logic of the column shards of the jitconn matmat: the ranges tile the columns, and rank r calls the
  unchanged operator with its width and the seed advanced by its first column (mod 2^32)."""
  from brainpylib_b200 import jitconn_ops
  calls = []

  def fake(matrix, *, kind, w1, w2, conn_prob, shape, seed, out=None):
    calls.append((shape, seed))
    return torch.zeros(matrix.shape[0], shape[1])

  monkeypatch.setattr(jitconn_ops, 'matmat_raw', fake)
  X = torch.zeros(4, 50)
  n, seed, world = 1003, 2 ** 32 - 100, 8
  outs = [sharded.matmat_column_shard(X, kind='normal', w1=0., w2=1., conn_prob=0.1, shape=(50, n), seed=seed,
                                      rank=r, world=world) for r in range(world)]
  assert sum(o.shape[1] for o in outs) == n
  lo = 0
  for (shape, s), o in zip(calls, outs):
    assert shape == (50, o.shape[1]) and s == (seed + lo) % 2 ** 32
    lo += o.shape[1]
  # more ranks than columns: the surplus ranks get an empty shard and make no call
  calls.clear()
  outs = [sharded.matmat_column_shard(X, kind='normal', w1=0., w2=1., conn_prob=0.1, shape=(50, 3), seed=1,
                                      rank=r, world=8) for r in range(8)]
  assert [o.shape[1] for o in outs] == [1, 1, 1, 0, 0, 0, 0, 0] and len(calls) == 3


# ------------------------------------------------------------------------------------------
# A wait that timed out on ONE rank must stop ALL ranks (that rank may overwrite slots its peers still read,
# and their own status words stay clean): check_all combines the status words over the process group.
# ------------------------------------------------------------------------------------------
def _status_worker(rank, world, port, failing_rank, out_queue):
  os.environ['MASTER_ADDR'] = '127.0.0.1'
  os.environ['MASTER_PORT'] = str(port)
  dist.init_process_group('gloo', rank=rank, world_size=world)
  try:
    ex = sharded.PushExchange.__new__(sharded.PushExchange)      # the host logic only: no device buffers
    ex.slots, ex.world, ex.rank = 4, world, rank
    ex._state = torch.zeros(4 + 1 + 32, dtype=torch.int32)
    if rank == failing_rank:
      ex._state[4] = 1                                           # what a timed-out wait leaves behind
    own = 'ok'
    try:
      ex.check()
    except RuntimeError:
      own = 'raised'
    combined = 'ok'
    try:
      ex.check_all()
    except RuntimeError:
      combined = 'raised'
    out_queue.put((rank, own, combined))
  finally:
    dist.destroy_process_group()


def test_a_timeout_on_one_rank_is_seen_by_every_rank():
  ctx = mp.get_context('spawn')
  for failing in (1, None):
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_status_worker, args=(r, 2, port, failing, q)) for r in range(2)]
    for p in procs:
      p.start()
    got = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
      p.join(timeout=60)
      assert p.exitcode == 0
    if failing is None:
      assert got == [(0, 'ok', 'ok'), (1, 'ok', 'ok')]
    else:
      assert got == [(0, 'ok', 'raised'), (1, 'raised', 'raised')]


def test_sharded_step_refuses_operands_it_would_index_out_of_bounds():
  ex = sharded.PushExchange.__new__(sharded.PushExchange)
  ex.n_events, ex.device = 100, torch.device('cpu')
  good = (torch.zeros(5), torch.zeros(5, dtype=torch.int32), torch.zeros(101, dtype=torch.int32))
  ex._check_matrix(*good)
  import pytest
  with pytest.raises(ValueError):
    ex._check_matrix(good[0], good[1], torch.zeros(100, dtype=torch.int32))          # one row pointer short
  with pytest.raises(TypeError):
    ex._check_matrix(good[0], good[1].to(torch.int64), good[2])
  with pytest.raises(ValueError):
    ex._check_matrix(torch.zeros(4), good[1], good[2])                               # weights / indices disagree
