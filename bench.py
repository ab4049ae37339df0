#!/usr/bin/env python
"""Benchmark of the synaptic-propagation hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload: the 1,000,000-neuron event-driven CSR step — 1e6 pre x 1e6 post neurons, 1000
outgoing synapses per neuron (1e9 stored synapses: 4 GB int32 indices + 4 GB float32 weights
U(0,1)), a fresh float32 spike vector per step with 1 % of the entries set (seeded numpy
PCG64 draws, `brainpylib_b200/workloads.py`), `event_csr_matvec(..., transpose=True)`.
One "step" = one call.  Metric: synaptic operations per second = (sum over the step's active
rows of the row length) / time, whole job.

Prints ONE JSON line (rank 0).  `value` is timed with the matrix, the spikes and the output
resident in HBM (CUDA graph of the K steps, CUDA events, max over ranks); `e2e` goes through
the public operator with host spike buffers in and host result buffers out every step;
`roofline` is for the scatter kernel alone (CUDA events recorded around it by the library's
profiling hook); `cpu_baseline` / `--impl reference` time the reference's own CPU kernel
(lib/cpu_event_sum.cc compiled into oracle/_ref, else this repository's CPU restatement).
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)

N_NEURONS = 1_000_000
DEGREE = 1000
CPU_SAMPLE_ROWS = 100_000   # rows of the matrix the CPU legs work on (the first generation chunk)
RATE = 0.01
METRIC = 'synaptic_ops_per_sec'
UNIT = 'SyOp/s'
WORKLOAD = 'C3 event_csr_matvec transpose=True: 1e6 neurons x 1000 synapses (1e9 nnz, heter f32 U(0,1)), ' \
           'f32 events 1% firing, fresh spikes every step'


def log(*a):
  print(*a, file=sys.stderr, flush=True)


def measured_peaks():
  path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
  if os.path.exists(path):
    try:
      return float(json.load(open(path))['hbm_gbs']), 'measured (MEASURED_PEAKS.json hbm_gbs)'
    except Exception:
      pass
  return 6650.0, 'fallback (6.65 TB/s, earlier measurement on this pool)'


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
  """Samples SM clock and throttle reasons through NVML while the GPU is busy."""

  def __init__(self, index):
    self.samples, self.reasons, self.max_mhz = [], set(), None
    self._stop = threading.Event()
    self._thread = None
    try:
      import pynvml
      pynvml.nvmlInit()
      self.nv = pynvml
      self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
      self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
    except Exception as e:   # NVML missing: report nothing rather than fail the run
      self.nv = None
      log(f'[bench] NVML unavailable: {e}')

  def _loop(self):
    nv = self.nv
    names = {
      'hw_slowdown': getattr(nv, 'nvmlClocksThrottleReasonHwSlowdown', 0x8),
      'hw_thermal_slowdown': getattr(nv, 'nvmlClocksThrottleReasonHwThermalSlowdown', 0x40),
      'sw_thermal_slowdown': getattr(nv, 'nvmlClocksThrottleReasonSwThermalSlowdown', 0x20),
      'sw_power_cap': getattr(nv, 'nvmlClocksThrottleReasonSwPowerCap', 0x4),
    }
    while not self._stop.is_set():
      try:
        util = nv.nvmlDeviceGetUtilizationRates(self.h).gpu
        mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
        mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        self.samples.append((mhz, util))
        for k, bit in names.items():
          if mask & bit:
            self.reasons.add(k)
      except Exception:
        pass
      time.sleep(0.002)

  def __enter__(self):
    if self.nv is not None:
      self._thread = threading.Thread(target=self._loop, daemon=True)
      self._thread.start()
    return self

  def __exit__(self, *exc):
    self._stop.set()
    if self._thread is not None:
      self._thread.join()

  def summary(self):
    if not self.samples:
      return {'sm_mhz': None, 'sm_max_mhz': self.max_mhz, 'reasons': [], 'samples': 0}
    busy = [m for m, u in self.samples if u > 0] or [m for m, _ in self.samples]
    return {'sm_mhz': float(np.median(busy)), 'sm_max_mhz': self.max_mhz, 'reasons': sorted(self.reasons),
            'samples': len(self.samples), 'samples_under_load': len(busy)}


# ------------------------------------------------------------------------------------------------
# workload
# ------------------------------------------------------------------------------------------------
def build_workload(n_steps, keep_host_matrix, device=None, shard=None, n_neurons=N_NEURONS):
  """The matrix on `device` (or only on the host) plus `n_steps` spike vectors (host, float32).

  `shard` = (rank, world): keep only the synapses whose target lies in this rank's contiguous
  range of post-synaptic neurons (own indptr), filtered on the GPU chunk by chunk.
  """
  from brainpylib_b200 import workloads
  import torch
  t0 = time.time()
  host = {'indices': [], 'data': []}
  dev = {'indices': [], 'data': []}
  lengths = []
  lo = hi = None
  if shard is not None:
    rank, world = shard
    per = (n_neurons + world - 1) // world
    lo, hi = rank * per, min(n_neurons, (rank + 1) * per)
  masks = []
  rng = None
  for kind, c, arr in workloads.c3_matrix_chunks(n_neurons):
    if kind == 'rng':
      rng = arr
      continue
    if keep_host_matrix and c == 0:
      host[kind].append(arr)     # the CPU legs run on the first 100,000 rows (chunk 0) only
    if device is not None:
      t = torch.from_numpy(arr).to(device, non_blocking=False)
      if shard is not None:
        if kind == 'indices':
          m = (t >= lo) & (t < hi)
          masks.append(m)
          lengths.append(m.view(-1, DEGREE).sum(dim=1, dtype=torch.int32))
          t = t[m] - lo
        else:
          t = t[masks[c]]
          masks[c] = None
      dev[kind].append(t)
  events = [workloads.c3_events(rng, n_neurons, RATE) for _ in range(n_steps)]
  out = {'events': events, 'gen_seconds': None}
  if device is not None:
    out['indices'] = torch.cat(dev['indices'])
    dev['indices'] = None
    out['data'] = torch.cat(dev['data'])
    dev['data'] = None
    if shard is None:
      out['indptr'] = torch.arange(0, n_neurons * DEGREE + 1, DEGREE, dtype=torch.int32, device=device)
      out['shape'] = (n_neurons, n_neurons)
    else:
      ptr = torch.zeros(n_neurons + 1, dtype=torch.int64, device=device)
      ptr[1:] = torch.cumsum(torch.cat(lengths).to(torch.int64), 0)
      out['indptr'] = ptr.to(torch.int32)
      out['shape'] = (n_neurons, hi - lo)
    torch.cuda.synchronize()
  if keep_host_matrix:
    out['host_indices'], out['host_data'] = host['indices'][0], host['data'][0]
    out['host_indptr'] = np.arange(0, CPU_SAMPLE_ROWS * DEGREE + 1, DEGREE, dtype=np.int32)
  out['gen_seconds'] = time.time() - t0
  return out


def workloads_chunk_rows():
  from brainpylib_b200 import workloads
  return workloads.C3_ROWS_PER_CHUNK


def cpu_reference_kernel():
  """(callable(events_f32) -> y, kind): the reference's own compiled CPU kernel when oracle/_ref
  holds it, else this repository's CPU restatement of it."""
  from oracle import ref
  if ref.available_cpu():
    return 'reference'
  return 'port'


CPU_SAMPLE = ('pre-synaptic rows 0..99,999 of the same matrix (1e8 synapses, all 1e6 post-synaptic targets) with '
              'the same spike vectors restricted to those rows: ~1e6 synaptic ops per step')


def time_cpu_steps(work, n_steps, budget_seconds=None):
  """Times the reference CPU path (serial C++: 1 core) on a bounded sample of the workload: the first
  100,000 rows of the matrix, every step's spikes restricted to those rows."""
  from oracle import cpu as oracle_cpu
  from oracle import ref
  kind = cpu_reference_kernel()
  ops, t_total, done = 0, 0.0, 0
  for s in range(n_steps):
    ev = work['events'][s % len(work['events'])][:CPU_SAMPLE_ROWS]
    if kind == 'reference':
      evb = ev != 0    # lib/cpu_event_sum.cc takes bool events; same truthiness test as the GPU op
      t0 = time.perf_counter()
      ref.csr_event_sum(evb, work['host_indices'], work['host_indptr'], work['host_data'], N_NEURONS)
      t_total += time.perf_counter() - t0
    else:
      t0 = time.perf_counter()
      oracle_cpu.event_csr_matvec(work['host_data'], work['host_indices'], work['host_indptr'], ev,
                                  shape=(CPU_SAMPLE_ROWS, N_NEURONS), transpose=True)
      t_total += time.perf_counter() - t0
    ops += int(np.count_nonzero(ev)) * DEGREE
    done += 1
    if budget_seconds is not None and t_total > budget_seconds:
      break
  return ops / t_total, kind, done, t_total


# ------------------------------------------------------------------------------------------------
# reference arm
# ------------------------------------------------------------------------------------------------
def run_reference(args):
  rank = int(os.environ.get('RANK', '0'))
  if rank != 0:
    return
  total = args.warmup + args.steps
  work = build_workload(total, keep_host_matrix=True, device=None)
  log(f'[bench] reference arm: host matrix built in {work["gen_seconds"]:.1f}s')
  if args.warmup:
    time_cpu_steps({**work, 'events': work['events'][:args.warmup]}, args.warmup)
  value, kind, done, seconds = time_cpu_steps({**work, 'events': work['events'][args.warmup:]}, args.steps)
  line = {
    'impl': 'reference', 'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': done,
    'warmup': args.warmup, 'ms_per_step': seconds / done * 1e3, 'higher_is_better': True, 'scaling': 'strong',
    'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
    'config': {'workload': WORKLOAD, 'reference_code': 'lib/cpu_event_sum.cc cpu_csr_event_sum_heter_f32_i32 '
               '(serial C++) on the host'},
    'cpu_baseline': {'value': value, 'unit': UNIT, 'cores': 1, 'kind': kind,
                     'sample': f'{done} steps on {CPU_SAMPLE}', 'host_cores_available': os.cpu_count()},
    'e2e': {'value': value, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
    'gpu_launches': 0,
  }
  print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args):
  import torch
  import torch.distributed as dist
  import brainpylib_b200 as bpl
  from brainpylib_b200 import _lib, event_ops, gpu_ops

  world = int(os.environ.get('WORLD_SIZE', '1'))
  rank = int(os.environ.get('RANK', '0'))
  local_rank = int(os.environ.get('LOCAL_RANK', '0'))
  if not torch.cuda.is_available():
    raise SystemExit('bench.py needs a CUDA device (no CPU fallback)')
  torch.cuda.set_device(local_rank)
  device = torch.device('cuda', local_rank)
  if world > 1:
    dist.init_process_group('nccl', device_id=device)
  _lib.lib()   # fail loudly if the CUDA library is missing

  K, W = args.steps, args.warmup
  total = W + K
  want_cpu = (world == 1 and rank == 0 and not args.no_cpu_baseline)
  n_neurons = args.neurons
  if n_neurons % workloads_chunk_rows() != 0 or n_neurons % world != 0:
    raise SystemExit('--neurons must be a multiple of 100000 and of the number of ranks')
  want_cpu = want_cpu and n_neurons == N_NEURONS
  work = build_workload(total, keep_host_matrix=want_cpu, device=device, shard=(rank, world) if world > 1 else None,
                        n_neurons=n_neurons)
  log(f'[bench] rank {rank}: workload built in {work["gen_seconds"]:.1f}s, '
      f'{work["indices"].numel():,} synapses on device')
  shape = work['shape']
  ops_per_step = [int(np.count_nonzero(e)) * DEGREE for e in work['events']]
  ev_host = torch.from_numpy(np.stack(work['events'])).pin_memory()
  ev_dev = ev_host.to(device)
  y = torch.empty(shape[1], dtype=torch.float32, device=device)
  name = 'event_csr_matvec_heter_float_float'
  opaque = gpu_ops.build_twouint_onebool_descriptor(shape[0], shape[1], True)
  ws = torch.empty(_lib.workspace_bytes(name, opaque), dtype=torch.uint8, device=device)

  # N > 1: every rank produces the spikes of its own 1/N of the neurons and the dense spike vector is
  # all-gathered (NCCL over NVLink) inside the step; the matrix shard then needs no further exchange.
  # The spikes of a step are inputs (they do not depend on the previous step's output), so inside the
  # captured graph the all-gather of step s+1 runs on a second stream while step s is scattered.
  per = n_neurons // world
  ev_full = [torch.empty(n_neurons, dtype=torch.float32, device=device) for _ in range(2)] if world > 1 else None
  comm_stream = torch.cuda.Stream(device) if world > 1 else None

  def compute(s, events, out=y):
    event_ops.event_csr_matvec_raw(work['data'], work['indices'], work['indptr'], events, shape=shape,
                                   transpose=True, out=out, workspace=ws)

  def step(s, out=y):
    events = ev_dev[s]
    if world > 1:
      dist.all_gather_into_tensor(ev_full[0], ev_dev[s, rank * per:(rank + 1) * per])
      events = ev_full[0]
    compute(s, events, out)

  def run_steps(first, count):
    """`count` steps on the current stream; with several ranks the gathers are double-buffered on
    `comm_stream` (event dependencies only, so the whole pattern can be captured in a graph)."""
    if world == 1:
      for s in range(first, first + count):
        compute(s, ev_dev[s])
      return
    if one_launch:
      mine = slice(rank * per, (rank + 1) * per)
      exchange.prime(ev_dev[first, mine], y_pair[0])
      for i in range(count):
        last = i == count - 1
        exchange.step(work['data'], work['indices'], work['indptr'], y_pair[i % 2],
                      None if last else y_pair[(i + 1) % 2], None if last else ev_dev[first + i + 1, mine])
      return
    main = torch.cuda.current_stream(device)
    gathered, consumed = {}, {}
    start = torch.cuda.Event()
    start.record(main)
    comm_stream.wait_event(start)
    for i in range(count):
      s = first + i
      b = i % (exchange.slots if exchange is not None else 2)
      with torch.cuda.stream(comm_stream):
        if i >= 2:
          comm_stream.wait_event(consumed[i - 2])     # at most one step of run-ahead
        if fused:
          exchange.push_compacted(ev_dev[s, rank * per:(rank + 1) * per], b)   # compaction + peer stores, one kernel
        elif exchange is not None:
          exchange.push(ev_dev[s, rank * per:(rank + 1) * per], b)     # peer stores over NVLink
        else:
          dist.all_gather_into_tensor(ev_full[b], ev_dev[s, rank * per:(rank + 1) * per])
        gathered[i] = torch.cuda.Event()
        gathered[i].record(comm_stream)
      main.wait_event(gathered[i])
      if fused:
        exchange.wait_zero(b, y)                      # bounded wait for every peer's list; zero-fills y
        exchange.scatter_from_list(work['data'], work['indices'], work['indptr'], b, y, shape[1])
      elif exchange is not None:
        exchange.wait(b)                              # bounded wait for every peer's slice
        compute(s, exchange.events(b))
      else:
        compute(s, ev_full[b])
      consumed[i] = torch.cuda.Event()
      consumed[i].record(main)
    done = torch.cuda.Event()
    done.record(comm_stream)
    main.wait_event(done)

  exchange = None
  if world > 1 and args.exchange in ('push', 'fused', 'step'):
    from brainpylib_b200 import sharded
    try:
      exchange = sharded.PushExchange(n_neurons, dtype=torch.float32, device=device, slots=4)
    except Exception as e:   # symmetric memory unavailable: keep the collective and say so
      log(f'[bench] rank {rank}: push exchange unavailable ({type(e).__name__}: {e}); using NCCL all-gather')
    ok = torch.tensor([1 if exchange is not None else 0], device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if not int(ok.item()):
      exchange = None
  fused = exchange is not None and args.exchange == 'fused'
  one_launch = exchange is not None and args.exchange == 'step'
  y_pair = [y, torch.empty_like(y)] if one_launch else None

  # sanity: one step against a plain torch scatter on the same device
  step(0)
  rows = torch.nonzero(ev_dev[0]).flatten()
  starts = work['indptr'][rows].to(torch.int64)
  lens = (work['indptr'][rows + 1] - work['indptr'][rows]).to(torch.int64)
  pos = torch.repeat_interleave(starts - torch.cumsum(lens, 0) + lens, lens) + torch.arange(int(lens.sum()),
                                                                                            device=device)
  chk = torch.zeros_like(y).index_add_(0, work['indices'][pos].to(torch.int64), work['data'][pos])
  err = (chk - y).abs().max().item()
  if not err < 1e-5 * 1000:
    raise SystemExit(f'bench sanity check failed: max abs error {err}')
  del rows, starts, lens, pos, chk

  sampler = ClockSampler(local_rank)
  with sampler:
    # ---- value: K steps captured in one CUDA graph, inputs resident in HBM ----
    side = torch.cuda.Stream(device)
    with torch.cuda.stream(side):
      for s in range(min(W, 3)):
        step(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
      run_steps(W, K)
    warm = torch.cuda.CUDAGraph()
    with torch.cuda.graph(warm, stream=side):
      run_steps(0, max(W, 1))
    if W:
      warm.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
      dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
      t = torch.tensor([ms], device=device)
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
      ms = t.item()
    total_ops = sum(ops_per_step[W:W + K])
    value = total_ops / (ms * 1e-3)
    if exchange is not None:
      exchange.check()                       # no wait timed out
      y_last = (y_pair[(K - 1) % 2] if one_launch else y).clone()
      step(W + K - 1)                        # same step through the NCCL path
      torch.cuda.synchronize()
      if not torch.allclose(y_last, y, rtol=1e-5, atol=1e-2):
        raise SystemExit('push exchange: result of the last step differs from the NCCL all-gather path')

    # ---- roofline: the scatter kernel alone, timed by events recorded around it ----
    lib = _lib.lib()
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    for s in range(K):
      a, b = pairs[s]
      a.record()   # creates the underlying CUDA events
      b.record()
    torch.cuda.synchronize()
    import ctypes
    for s in range(K):
      a, b = pairs[s]
      lib.bpl_profile_scatter_events(ctypes.c_void_p(a.cuda_event), ctypes.c_void_p(b.cuda_event))
      step(W + s)
    lib.bpl_profile_scatter_events(None, None)
    torch.cuda.synchronize()
    k_ms = float(np.mean([a.elapsed_time(b) for a, b in pairs]))

    # ---- e2e: public operator, host spikes in, host result out, every step ----
    e2e = run_e2e(torch, bpl, work, ev_host, shape, W, K, device, ops_per_step)
    if world > 1:
      t = torch.tensor([e2e['ms']], device=device)
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
      e2e['ms'] = t.item()
    e2e_value = total_ops / (e2e['ms'] * 1e-3)

    # ---- the same steps on the column-blocked format (converted once, outside any timed region) ----
    blocked = None
    if world == 1 and not args.no_blocked:
      t0 = time.time()
      cb = event_ops.csr_to_column_blocked(work['data'], work['indices'], work['indptr'], shape=shape)
      torch.cuda.synchronize()
      convert_s = time.time() - t0
      yb = torch.empty(shape[1], dtype=torch.float32, device=device)
      event_ops.event_cbcsr_matvec_raw(cb, ev_dev[0], out=yb)
      compute(0, ev_dev[0])
      torch.cuda.synchronize()
      cb_err = (yb - y).abs().max().item()
      if not cb_err < 1e-5 * 1000:
        raise SystemExit(f'column-blocked result differs from the CSR result: max abs error {cb_err}')
      g2 = torch.cuda.CUDAGraph()
      with torch.cuda.graph(g2, stream=side):
        for s in range(W, W + K):
          event_ops.event_cbcsr_matvec_raw(cb, ev_dev[s], out=yb)
      g2.replay()
      torch.cuda.synchronize()
      b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      b0.record()
      g2.replay()
      b1.record()
      torch.cuda.synchronize()
      cb_ms = b0.elapsed_time(b1)
      n_act_cb = float(np.mean([o / DEGREE for o in ops_per_step[W:W + K]]))
      # algorithmic bytes of a step in this format: 6 B per active synapse (16-bit id + weight), the block
      # offsets of every active row, spike scan, zero-fill and write-back of y
      cb_bytes = 6.0 * n_act_cb * DEGREE + 4.0 * n_act_cb * (cb.n_blocks + 1) + 4.0 * n_neurons + 8.0 * shape[1]
      hbm_peak = measured_peaks()[0]
      blocked = {'format': 'column-blocked CSR (event_cbcsr_matvec), converted once per matrix',
                 'value': sum(ops_per_step[W:W + K]) / (cb_ms * 1e-3), 'unit': UNIT, 'ms_per_step': cb_ms / K,
                 'block_width': cb.block_width, 'n_blocks': cb.n_blocks, 'convert_seconds': convert_s,
                 'format_bytes': cb.nbytes(), 'max_abs_diff_vs_csr': cb_err,
                 'roofline_step': {'algorithmic_bytes': cb_bytes, 'achieved': cb_bytes / (cb_ms / K * 1e-3) / 1e9,
                                   'frac': cb_bytes / (cb_ms / K * 1e-3) / 1e9 / hbm_peak, 'unit': 'GB/s'}}
      del cb, g2

  peak, peak_src = measured_peaks()
  n_act = float(np.mean([o / DEGREE for o in ops_per_step[W:W + K]]))
  s_local = float(work['indices'].numel()) / (n_neurons * DEGREE) * n_act * DEGREE   # this rank's synapses per step
  # algorithmic bytes of one scatter launch: indices + weights of the active rows (8 B per synapse),
  # their indptr pairs (8 B per active row) and the write-back of y (4 B per output neuron)
  k_bytes = 8.0 * s_local + 8.0 * n_act + 4.0 * shape[1]
  # whole step: + the spike scan (4 B per pre neuron) and the zero-fill of y (4 B per output neuron)
  step_bytes = k_bytes + 4.0 * n_neurons + 4.0 * shape[1]
  achieved = k_bytes / (k_ms * 1e-3) / 1e9
  roofline = {
    'bound': 'hbm', 'kernel': 'row_scatter_kernel<float, heter, list, vec>', 'achieved': achieved, 'peak': peak,
    'unit': 'GB/s', 'frac': achieved / peak, 'peak_source': peak_src,
    # DRAM bytes per launch: an ncu capture of this kernel on a 4e5-neuron twin read 1.046x its algorithmic
    # bytes (profiles/row_scatter_kernel_c3_event_csr.md); traffic grows with the active synapses
    'traffic': 1.046 * k_bytes, 'traffic_source': 'ncu dram__bytes on a reduced twin, scaled by algorithmic bytes',
    'algorithmic_bytes_per_launch': k_bytes, 'kernel_us': k_ms * 1e3,
    'step': {'algorithmic_bytes': step_bytes, 'us': ms / K * 1e3,
             'frac': step_bytes / (ms / K * 1e-3) / 1e9 / peak},
  }

  line = {
    'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': K, 'warmup': W,
    'ms_per_step': ms / K, 'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32',
    'data': 'synthetic',
    'config': {'workload': WORKLOAD if n_neurons == N_NEURONS else
               f'REDUCED TWIN of C3 for profiler captures: {n_neurons} neurons x 1000 synapses (not the benchmark size)',
               'l2': 'inputs larger than L2: each step streams a different ~80 MB of the '
               '8 GB matrix; spikes and output (4 MB each) are L2-resident by design',
               'sharding': 'none' if world == 1 else f'post-synaptic neurons (matrix columns) split over {world} '
               'ranks; each rank owns 1/N of the spike sources; every step the dense spike vector is assembled by '
               + ('ONE launch per step: the kernel pushes the compacted spikes of step s+1 into every peer over NVLink, waits '
                  '(bounded) for the lists of step s and scatters them' if one_launch else
                  "one kernel that compacts the rank's own spikes and stores the list into every peer over NVLink, bounded waits"
                  if fused else 'peer stores over NVLink with bounded waits (push exchange)' if exchange is not None
                  else 'an NCCL all-gather')
               + ('' if one_launch else ', one step ahead on a second stream (step s+1 is exchanged while step s scatters)')},
    'e2e': {'value': e2e_value, 'unit': UNIT, 'h2d_bytes_per_step': e2e['h2d'], 'd2h_bytes_per_step': e2e['d2h'],
            'ms_per_step': e2e['ms'] / K},
    # own kernels in the timed graph: scan + scatter per step; push, wait, scan + scatter (dense push);
    # push, wait, scatter (fused); prime once then one kernel per step (step)
    'gpu_launches': (K + 1 if one_launch else 3 * K if fused else 4 * K if exchange is not None else 2 * K),
    'roofline': roofline,
    'clocks': sampler.summary(),
  }

  if blocked is not None:
    line['column_blocked'] = blocked
  if want_cpu:
    cpu_value, kind, done, seconds = time_cpu_steps(work, 100000, budget_seconds=10.0)
    line['cpu_baseline'] = {'value': cpu_value, 'unit': UNIT, 'cores': 1, 'kind': kind,
                            'sample': f'{done} steps ({seconds:.1f} s of CPU time) on {CPU_SAMPLE}; '
                                      'lib/cpu_event_sum.cc serial C++',
                            'host_cores_available': os.cpu_count()}
  if rank == 0:
    print(json.dumps(line), flush=True)
  if world > 1:
    # Tear down in a fixed order: the captured graphs hold NCCL kernels and must go before the
    # communicator.  A process that still cannot finish the teardown within 30 s leaves anyway:
    # the measurement is complete and printed, and a launcher must not wait on it for ever.
    sys.stdout.flush()
    sys.stderr.flush()
    watchdog = threading.Timer(30.0, lambda: os._exit(0))
    watchdog.daemon = True
    watchdog.start()
    torch.cuda.synchronize()
    dist.barrier()
    graph.reset()
    warm.reset()
    torch.cuda.synchronize()
    dist.destroy_process_group()
    watchdog.cancel()


def run_e2e(torch, bpl, work, ev_host, shape, W, K, device, ops_per_step):
  """End to end through the C ABI with HOST buffers: every step copies that step's spike vector from
  pinned host memory to the device, calls the custom-call target, and copies the result back to pinned
  host memory.  Three streams (copy in, compute, copy out) and triple buffers, so step s+1's spikes are
  copied in while step s computes and step s-1's result is copied out.  The CUDA runtime is driven
  directly (ctypes) so that Python dispatch stays off the critical path."""
  import ctypes
  from brainpylib_b200 import _lib, gpu_ops
  rt = ctypes.CDLL('libcudart.so.12')
  rt.cudaMemcpyAsync.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
  rt.cudaEventCreateWithFlags.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_uint]
  rt.cudaEventRecord.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
  rt.cudaStreamWaitEvent.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint]

  def check(code):
    if code != 0:
      raise SystemExit(f'CUDA runtime call failed with error {code}')

  streams = [torch.cuda.Stream(device) for _ in range(3)]
  s_in, s_c, s_out = (ctypes.c_void_p(st.cuda_stream) for st in streams)
  n_buf = 3
  ev_buf = [torch.empty(shape[0], dtype=torch.float32, device=device) for _ in range(n_buf)]
  y_buf = [torch.empty(shape[1], dtype=torch.float32, device=device) for _ in range(n_buf)]
  y_host = [torch.empty(shape[1], dtype=torch.float32).pin_memory() for _ in range(n_buf)]
  name = 'event_csr_matvec_heter_float_float'
  opaque = gpu_ops.build_twouint_onebool_descriptor(shape[0], shape[1], True)
  ws = torch.empty(_lib.workspace_bytes(name, opaque), dtype=torch.uint8, device=device)
  target = _lib.target(name)
  bufs = [(ctypes.c_void_p * 6)(work['data'].data_ptr(), work['indices'].data_ptr(), work['indptr'].data_ptr(),
                                ev_buf[b].data_ptr(), y_buf[b].data_ptr(), ws.data_ptr()) for b in range(n_buf)]

  def new_event():
    e = ctypes.c_void_p()
    check(rt.cudaEventCreateWithFlags(ctypes.byref(e), 2))   # cudaEventDisableTiming
    return e
  done_in, done_c, done_out = ([new_event() for _ in range(n_buf)] for _ in range(3))
  used = [False] * n_buf
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  h2d, d2h = 4 * shape[0], 4 * shape[1]

  def run(first, count, timed):
    torch.cuda.synchronize()
    for b in range(n_buf):
      used[b] = False
    if timed:
      e0.record(streams[0])
    for i in range(count):
      s, b = first + i, i % n_buf
      if used[b]:
        check(rt.cudaStreamWaitEvent(s_in, done_c[b], 0))      # the spike buffer's previous reader has finished
        check(rt.cudaStreamWaitEvent(s_c, done_out[b], 0))     # the result buffer's previous copy-out has finished
      check(rt.cudaMemcpyAsync(ev_buf[b].data_ptr(), ev_host[s].data_ptr(), h2d, 1, s_in))
      check(rt.cudaEventRecord(done_in[b], s_in))
      check(rt.cudaStreamWaitEvent(s_c, done_in[b], 0))
      target(s_c, bufs[b], opaque, len(opaque))
      check(rt.cudaEventRecord(done_c[b], s_c))
      check(rt.cudaStreamWaitEvent(s_out, done_c[b], 0))
      check(rt.cudaMemcpyAsync(y_host[b].data_ptr(), y_buf[b].data_ptr(), d2h, 2, s_out))
      check(rt.cudaEventRecord(done_out[b], s_out))
      used[b] = True
    _lib.check_status()
    if timed:
      streams[2].wait_stream(streams[1])
      e1.record(streams[2])
    torch.cuda.synchronize()

  run(0, max(W, 1), False)
  run(W, K, True)
  # the last result that reached the host is the last step's
  last = (K - 1) % n_buf
  if not torch.isfinite(y_host[last]).all() or float(y_host[last].abs().sum()) == 0.0:
    raise SystemExit('e2e: the result copied back to the host is empty')
  return {'ms': e0.elapsed_time(e1), 'h2d': h2d, 'd2h': d2h}


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument('--gpus', type=int, default=1)
  ap.add_argument('--steps', type=int, default=200)
  ap.add_argument('--warmup', type=int, default=5)
  ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
  ap.add_argument('--no-cpu-baseline', action='store_true')
  ap.add_argument('--no-blocked', action='store_true', help='skip the column-blocked format measurement')
  ap.add_argument('--exchange', default='step', choices=['step', 'fused', 'push', 'nccl'],
                  help='N > 1: how the spikes reach every rank each step: step (one launch per step: push of the next step fused with this step scatter), fused (compaction + peer stores of spike lists), '
                  'push (peer stores of the dense slice) or nccl (all-gather)')
  ap.add_argument('--config', default='c3', choices=['c1', 'c2', 'c3', 'c4', 'c5'],
                  help='c3 (default) is the benchmark; the other configurations print their own JSON lines '
                       '(1 GPU, see brainpylib_b200/config_bench.py)')
  ap.add_argument('--neurons', type=int, default=N_NEURONS,
                  help='reduced twin of the workload (multiple of 100000), for profiler captures only')
  args = ap.parse_args()
  if args.warmup < 3 and args.impl == 'ours':
    log('[bench] note: fewer than 3 warm-up steps requested; the timing rules ask for >= 3')
  if args.config != 'c3':
    from brainpylib_b200 import config_bench
    return config_bench.main([args.config, '--warmup', str(args.warmup)])
  if args.impl == 'reference':
    run_reference(args)
  else:
    run_ours(args)


if __name__ == '__main__':
  main()
