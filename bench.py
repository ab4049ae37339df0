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

Prints ONE JSON line (rank 0).

1 GPU.  `value`: `event_csr_matvec(..., transpose=True, prepared=...)`: the public operator on the matrix
prepared once into the column-blocked layout (float32 accumulation), K steps in one CUDA graph, inputs
resident in HBM, CUDA events.  `stateless_csr` is the same operator without the prepared matrix (the
reference's exact signature), `prepared_fixed_point` the prepared matrix with fixed-point accumulation.
`roofline` is for the dominant kernel of `value` alone (CUDA events recorded around it by the library's
profiling hook).  `e2e` drives the C-ABI target with HOST buffers (`HostSteps`, `bpl_run_host_steps`): every step
copies that step's spikes from pinned host memory and the result back, three streams, enqueued by native code.
N > 1 GPUs.  The matrix is sharded by post-synaptic neuron (shards prepared like the 1-GPU matrix while a rank keeps
>= 200,000 columns, plain CSR below: sharded.preferred_layout), every rank owns 1/N of the
spike sources, one launch per step pushes the next step's spike list to the peers and scatters this
step's; `e2e` moves only the rank's own n/N spikes in and its own slice of the result out.
`cpu_baseline` / `--impl reference` time the reference's own CPU kernel (lib/cpu_event_sum.cc compiled
into oracle/_ref, else this repository's CPU restatement) on the FULL matrix, same spikes.
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
RATE = 0.01
METRIC = 'synaptic_ops_per_sec'
UNIT = 'SyOp/s'
WORKLOAD = 'C3 event_csr_matvec transpose=True: 1e6 neurons x 1000 synapses (1e9 nnz, heter f32 U(0,1)), ' \
           'f32 events 1% firing, fresh spikes every step'


def log(*a):
  print(*a, file=sys.stderr, flush=True)


_RESULT_OUT = None


def keep_stdout_for_the_result():
  """Libraries loaded later (NCCL's version banner) write to file descriptor 1: point it at stderr and keep the
  original for the one JSON line."""
  global _RESULT_OUT
  if _RESULT_OUT is None:
    sys.stdout.flush()
    _RESULT_OUT = os.fdopen(os.dup(1), 'w')
    os.dup2(2, 1)


def emit(line):
  out = _RESULT_OUT if _RESULT_OUT is not None else sys.stdout
  out.write(json.dumps(line) + '\n')
  out.flush()


def measured_peaks():
  path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
  if os.path.exists(path):
    try:
      return float(json.load(open(path))['hbm_gbs']), 'measured (MEASURED_PEAKS.json hbm_gbs)'
    except Exception:
      pass
  return 6650.0, 'fallback (6.65 TB/s: MEASURED_PEAKS.json is absent)'


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
    if keep_host_matrix:
      host[kind].append(arr)     # the CPU legs run on the whole matrix (8 GB of host memory)
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
    out['host_indices'], out['host_data'] = np.concatenate(host['indices']), np.concatenate(host['data'])
    host.clear()
    out['host_indptr'] = np.arange(0, n_neurons * DEGREE + 1, DEGREE, dtype=np.int32)
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


CPU_SAMPLE = 'the whole 1e6 x 1e6 matrix (1e9 synapses) on the host, the same spike vectors: ~1e7 synaptic ops per step'


def time_cpu_steps(work, n_steps, budget_seconds=None):
  """Times the reference CPU path (serial C++: 1 core) on the whole matrix, step after step, until the
  steps or the time budget run out."""
  from oracle import cpu as oracle_cpu
  from oracle import ref
  kind = cpu_reference_kernel()
  ops, t_total, done = 0, 0.0, 0
  for s in range(n_steps):
    ev = work['events'][s % len(work['events'])]
    if kind == 'reference':
      evb = ev != 0    # lib/cpu_event_sum.cc takes bool events; same truthiness test as the GPU op
      t0 = time.perf_counter()
      ref.csr_event_sum(evb, work['host_indices'], work['host_indptr'], work['host_data'], N_NEURONS)
      t_total += time.perf_counter() - t0
    else:
      t0 = time.perf_counter()
      oracle_cpu.event_csr_matvec(work['host_data'], work['host_indices'], work['host_indptr'], ev,
                                  shape=(N_NEURONS, N_NEURONS), transpose=True)
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
  emit(line)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def graph_time_ms(torch, device, side, fn, first, count, warm_first, warm_count):
  """Milliseconds of `count` calls fn(s) captured in one CUDA graph (CUDA events around one replay), after a
  replay of a warm-up graph of `warm_count` calls.  Returns (ms, graph, warm_graph)."""
  graph, warm = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
  with torch.cuda.graph(graph, stream=side):
    for s in range(first, first + count):
      fn(s)
  with torch.cuda.graph(warm, stream=side):
    for s in range(warm_first, warm_first + max(warm_count, 1)):
      fn(s)
  warm.replay()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  torch.cuda.synchronize()
  e0.record()
  graph.replay()
  e1.record()
  torch.cuda.synchronize()
  return e0.elapsed_time(e1), graph, warm


def kernel_time_ms(torch, lib, fn, first, count):
  """Mean milliseconds of the scatter kernel alone over `count` calls fn(s), from the events the library
  records directly around it."""
  import ctypes
  pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(count)]
  for a, b in pairs:
    a.record()   # creates the underlying CUDA events
    b.record()
  torch.cuda.synchronize()
  for i, (a, b) in enumerate(pairs):
    lib.bpl_profile_scatter_events(ctypes.c_void_p(a.cuda_event), ctypes.c_void_p(b.cuda_event))
    fn(first + i)
  lib.bpl_profile_scatter_events(None, None)
  torch.cuda.synchronize()
  return float(np.mean([a.elapsed_time(b) for a, b in pairs]))


def torch_reference_step(torch, work, events, n_out):
  """y of one step by a plain torch scatter on the same device (an independent computation)."""
  rows = torch.nonzero(events).flatten()
  starts = work['indptr'][rows].to(torch.int64)
  lens = (work['indptr'][rows + 1] - work['indptr'][rows]).to(torch.int64)
  pos = torch.repeat_interleave(starts - torch.cumsum(lens, 0) + lens, lens) + torch.arange(int(lens.sum()),
                                                                                            device=events.device)
  return torch.zeros(n_out, dtype=torch.float32, device=events.device).index_add_(
    0, work['indices'][pos].to(torch.int64), work['data'][pos])


def run_ours(args):
  import torch
  import torch.distributed as dist
  from brainpylib_b200 import _lib
  world = int(os.environ.get('WORLD_SIZE', '1'))
  local_rank = int(os.environ.get('LOCAL_RANK', '0'))
  if not torch.cuda.is_available():
    raise SystemExit('bench.py needs a CUDA device (no CPU fallback)')
  torch.cuda.set_device(local_rank)
  device = torch.device('cuda', local_rank)
  if world > 1:
    dist.init_process_group('nccl', device_id=device)
  _lib.lib()   # fail loudly if the CUDA library is missing
  if args.neurons % workloads_chunk_rows() != 0 or args.neurons % world != 0:
    raise SystemExit('--neurons must be a multiple of 100000 and of the number of ranks')
  if world == 1 and args.one_rank_of > 1:
    run_one_rank_of(args, torch, device)
  elif world == 1:
    run_single(args, torch, device)
  else:
    run_sharded(args, torch, dist, device, world)


def run_one_rank_of(args, torch, device):
  """Profiler aid, not a benchmark result: ONE process stands in for rank 0 of `--one-rank-of N` ranks.  It holds
  that rank's shard of the matrix (columns 0 .. n/N, prepared) and runs the one-launch sharded step on an exchange
  of world size 1.  Every step is primed separately (the prime call pushes all n spike sources, which N ranks would
  share) and the step launch itself pushes nothing, so the launch that is timed and captured is the scatter half of
  a rank's step: bounded poll, scatter of the assembled list on the 1/N shard, exit ticket.  Prints one JSON line
  marked as a profiler aid."""
  from brainpylib_b200 import event_ops, sharded
  K, W = args.steps, args.warmup
  n = args.neurons
  work = build_workload(W + K, keep_host_matrix=False, device=device, shard=(0, args.one_rank_of), n_neurons=n)
  shape = work['shape']
  prepared = event_ops.csr_to_column_blocked(work['data'], work['indices'], work['indptr'], shape=shape,
                                             block_width=event_ops.default_block_width(shape[1], device, reserve=4))
  ev = [torch.from_numpy(e).to(device) for e in work['events']]
  exchange = sharded.PushExchange(n, dtype=torch.float32, device=device, slots=4)
  y = [torch.empty(shape[1], dtype=torch.float32, device=device) for _ in range(2)]
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

  def run(first, count):
    total = 0.0
    for i in range(count):
      exchange.prime(ev[first + i], y[i % 2])
      e0.record()
      exchange.step_prepared(prepared, y[i % 2], None, None)
      e1.record()
      torch.cuda.synchronize()
      total += e0.elapsed_time(e1)
    exchange.check()
    return total

  run(0, max(W, 1))
  ms = run(W, K)
  emit({'profiler_aid': f'one process standing in for rank 0 of {args.one_rank_of}: scatter half of the step', 'n_gpus': 1,
        'steps': K, 'ms_per_step': ms / K, 'shard_columns': shape[1], 'synapses_on_device': int(work['indices'].numel()),
        'block_width': prepared.block_width, 'n_blocks': prepared.n_blocks})


def run_single(args, torch, device):
  import brainpylib_b200 as bpl
  from brainpylib_b200 import _lib, event_ops, gpu_ops
  K, W = args.steps, args.warmup
  n_neurons = args.neurons
  want_cpu = (not args.no_cpu_baseline) and n_neurons == N_NEURONS
  work = build_workload(W + K, keep_host_matrix=want_cpu, device=device, n_neurons=n_neurons)
  log(f'[bench] workload built in {work["gen_seconds"]:.1f}s, {work["indices"].numel():,} synapses on device')
  shape = work['shape']
  ops_per_step = [int(np.count_nonzero(e)) * DEGREE for e in work['events']]
  total_ops = sum(ops_per_step[W:W + K])
  n_act = float(np.mean([o / DEGREE for o in ops_per_step[W:W + K]]))
  ev_host = torch.from_numpy(np.stack(work['events'])).pin_memory()
  ev_dev = ev_host.to(device)
  y = torch.empty(shape[1], dtype=torch.float32, device=device)
  lib = _lib.lib()
  peak, peak_src = measured_peaks()

  # the matrix prepared once (outside every timed region): column-blocked layout, float and fixed-point accumulation
  prepared, convert_s = {}, {}
  for mode in ('float', 'fixed'):
    torch.cuda.synchronize()
    t0 = time.time()
    prepared[mode] = bpl.prepare_event_csr(work['data'], work['indices'], work['indptr'], shape=shape, accumulate=mode)
    torch.cuda.synchronize()
    convert_s[mode] = time.time() - t0
  cb = prepared['float']

  name_csr = 'event_csr_matvec_heter_float_float'
  opaque_csr = gpu_ops.build_twouint_onebool_descriptor(shape[0], shape[1], True)
  ws = torch.empty(_lib.workspace_bytes(name_csr, opaque_csr), dtype=torch.uint8, device=device)

  def raw_csr(s):
    event_ops.event_csr_matvec_raw(work['data'], work['indices'], work['indptr'], ev_dev[s], shape=shape,
                                   transpose=True, out=y, workspace=ws)

  def raw_prepared(mode):
    return lambda s: event_ops.event_cbcsr_matvec_raw(prepared[mode], ev_dev[s], out=y, workspace=ws)

  # sanity: the three paths against a plain torch scatter on the same device (through the public operator)
  chk = torch_reference_step(torch, work, ev_dev[0], shape[1])
  errs = {}
  for label, kw in (('stateless_csr', {}), ('prepared', {'prepared': prepared['float']}),
                    ('prepared_fixed_point', {'prepared': prepared['fixed']})):
    out = bpl.event_csr_matvec(work['data'], work['indices'], work['indptr'], ev_dev[0], shape=shape, transpose=True, **kw)
    errs[label] = (chk - out).abs().max().item()
    if not errs[label] < 1e-5 * DEGREE:
      raise SystemExit(f'bench sanity check failed ({label}): max abs error {errs[label]}')
  del chk, out

  sampler = ClockSampler(device.index)
  side = torch.cuda.Stream(device)
  with sampler:
    with torch.cuda.stream(side):
      for s in range(min(W, 3)):
        raw_csr(s)
        raw_prepared('float')(s)
        raw_prepared('fixed')(s)
    torch.cuda.synchronize()
    # ---- value: K steps captured in one CUDA graph, inputs resident in HBM ----
    ms, g_a, g_b = graph_time_ms(torch, device, side, raw_prepared('float'), W, K, 0, W)
    k_ms = kernel_time_ms(torch, lib, raw_prepared('float'), W, K)
    ms_csr, g_c, g_d = graph_time_ms(torch, device, side, raw_csr, W, K, 0, W)
    k_ms_csr = kernel_time_ms(torch, lib, raw_csr, W, K)
    ms_fix, g_e, g_f = graph_time_ms(torch, device, side, raw_prepared('fixed'), W, K, 0, W)
    k_ms_fix = kernel_time_ms(torch, lib, raw_prepared('fixed'), W, K)
    # ---- e2e: the C-ABI target with host buffers, every step ----
    e2e = run_e2e_single(torch, work, ev_host, shape, W, K, device, cb)
    fusion = caller_fusion(torch, device, side, prepared['fixed'], shape, K)
  value = total_ops / (ms * 1e-3)

  # algorithmic bytes of one scatter launch on the prepared matrix: 6 B per active synapse (weight + 16-bit id),
  # the two segment offsets every CTA column reads per active row (8 B x blocks), write-back of y (4 B per neuron)
  cb_kernel_bytes = 6.0 * n_act * DEGREE + 8.0 * n_act * cb.n_blocks + 4.0 * shape[1]
  # whole step: + the spike scan (4 B per pre neuron) and the zero-fill of y (4 B per output neuron)
  cb_step_bytes = cb_kernel_bytes + 4.0 * n_neurons + 4.0 * shape[1]
  csr_kernel_bytes = 8.0 * n_act * DEGREE + 8.0 * n_act + 4.0 * shape[1]
  csr_step_bytes = csr_kernel_bytes + 4.0 * n_neurons + 4.0 * shape[1]

  def roof(kernel, kbytes, kms, sbytes, sms, traffic_ratio, traffic_src):
    return {'bound': 'hbm', 'kernel': kernel, 'achieved': kbytes / (kms * 1e-3) / 1e9, 'peak': peak, 'unit': 'GB/s',
            'frac': kbytes / (kms * 1e-3) / 1e9 / peak, 'peak_source': peak_src,
            'traffic': traffic_ratio * kbytes if traffic_ratio else None, 'traffic_source': traffic_src,
            'algorithmic_bytes_per_launch': kbytes, 'kernel_us': kms * 1e3,
            'step': {'algorithmic_bytes': sbytes, 'us': sms / K * 1e3, 'frac': sbytes / (sms / K * 1e-3) / 1e9 / peak}}

  padded = prepared['float'].n_groups * 8 / float(work['indices'].numel())
  line = {
    'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': 1, 'steps': K, 'warmup': W, 'ms_per_step': ms / K,
    'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
    'config': {'workload': WORKLOAD if n_neurons == N_NEURONS else
               f'REDUCED TWIN of C3 for profiler captures: {n_neurons} neurons x 1000 synapses (not the benchmark size)',
               'path': 'event_csr_matvec(data, indices, indptr, events, shape=, transpose=True, prepared=P): P = '
                       'prepare_event_csr(...) once per matrix (column-blocked layout, float32 accumulation); '
                       'the same call without prepared= is reported under stateless_csr',
               'l2': 'inputs larger than L2: each step streams a different ~70 MB of the 6.9 GB prepared matrix '
                     '(~80 MB of the 8 GB CSR matrix); spikes and output (4 MB each) are L2-resident by design',
               'sharding': 'none'},
    'e2e': {'value': total_ops / (e2e['ms'] * 1e-3), 'unit': UNIT, 'h2d_bytes_per_step': e2e['h2d'],
            'd2h_bytes_per_step': e2e['d2h'], 'ms_per_step': e2e['ms'] / K,
            'path': 'brainpylib_b200.HostSteps.run -> bpl_run_host_steps -> C-ABI target event_cbcsr_matvec_heter_float_float: '
                    'pinned host spikes in, pinned host result out, every step'},
    'gpu_launches': 2 * K,     # spike scan + scatter per step
    'roofline': roof('event_cb_scatter_kernel<float accumulate>', cb_kernel_bytes, k_ms, cb_step_bytes, ms,
                     1.14,
                     'ncu dram__bytes of the same kernel on a reduced twin (4e5 neurons), scaled by algorithmic bytes; the '
                     'factor is the padding of records to 8 synapses'),
    'prepared_matrix': {'block_width': cb.block_width, 'n_blocks': cb.n_blocks, 'bytes': cb.nbytes(),
                        'csr_bytes': 8 * work['indices'].numel() + 4 * (n_neurons + 1),
                        'padding_factor': padded, 'convert_seconds': convert_s['float'],
                        'convert_seconds_fixed_point': convert_s['fixed'],
                        'scale_log2_fixed_point': prepared['fixed'].scale_log2},
    'stateless_csr': {'value': total_ops / (ms_csr * 1e-3), 'unit': UNIT, 'ms_per_step': ms_csr / K,
                      'roofline': roof('row_scatter_kernel<float, heter, list, vec>', csr_kernel_bytes, k_ms_csr,
                                       csr_step_bytes, ms_csr, 1.046,
                                       'ncu dram__bytes on a reduced twin, scaled by algorithmic bytes')},
    'prepared_fixed_point': {'value': total_ops / (ms_fix * 1e-3), 'unit': UNIT, 'ms_per_step': ms_fix / K,
                             'roofline': roof('event_cb_scatter_kernel<fixed-point accumulate>', cb_kernel_bytes,
                                              k_ms_fix, cb_step_bytes, ms_fix, None, None)},
    'max_abs_error_vs_torch_scatter': errs,
    'caller_fusion': fusion,
    'clocks': sampler.summary(),
  }
  line['reference_cuda'] = reference_cuda_c3(torch, work, ev_dev, shape, W, min(K, 20), ops_per_step)
  if want_cpu:
    cpu_value, kind, done, seconds = time_cpu_steps(work, K, budget_seconds=15.0)
    line['cpu_baseline'] = {'value': cpu_value, 'unit': UNIT, 'cores': 1, 'kind': kind,
                            'sample': f'{done} steps ({seconds:.1f} s of CPU time) on {CPU_SAMPLE}; '
                                      'lib/cpu_event_sum.cc serial C++',
                            'host_cores_available': os.cpu_count()}
  emit(line)


def caller_fusion(torch, device, side, prepared, shape, K):
  """The closed simulation loop with the caller's side fused: per step ONE launch that decays the conductances,
  integrates the neurons, thresholds and compacts the new spikes (lif_exp_step_float) and ONE list-driven scatter on
  the prepared matrix; no spike vector is scanned and the output needs no zero-fill.  The neurons are driven so that
  1 % of them fire per step whatever the network does (membrane resistance 0: the synaptic input is accumulated but
  does not move the potentials; constant drive, uniformly spread phases, period 100 steps), which keeps the load equal
  to the benchmark's.  Synaptic operations are counted from the spikes of an identical untimed run."""
  import brainpylib_b200 as bpl
  from brainpylib_b200 import neuron_ops
  n = shape[0]
  period = 100
  p = neuron_ops.LifExpParams(dt=20.0 * np.log(2.0) / period, tau_syn=[5.0], E_rev=[0.0], ext_input=0.0, V_rest=-40.0,
                              V_th=-50.0, V_reset=-60.0, R=0.0, tau=20.0, tau_ref=-1.0)
  rng = np.random.default_rng(11)
  phase = rng.random(n)
  V0 = torch.as_tensor((-40.0 - 20.0 * np.power(0.5, phase)).astype(np.float32)).to(device)
  state = dict(V=V0.clone(), g=torch.zeros(n, device=device), y=torch.zeros(n, device=device),
               tl=torch.full((n,), -1e7, device=device))
  spikes = torch.empty(n, dtype=torch.float32, device=device)
  lst = torch.empty(neuron_ops.spike_list_bytes(n), dtype=torch.uint8, device=device)

  def step():
    bpl.lif_exp_step(state['y'], state['g'], state['V'], state['tl'], p, 0.0, spikes=spikes, spike_list=lst)
    bpl.event_csr_matvec_from_list(None, None, None, lst, state['y'], shape=shape, prepared=prepared)

  def reset():
    state['V'].copy_(V0)
    state['g'].zero_()
    state['y'].zero_()

  with torch.cuda.stream(side):
    for _ in range(3):
      step()
  torch.cuda.synchronize()
  graph = torch.cuda.CUDAGraph()
  with torch.cuda.graph(graph, stream=side):
    for _ in range(K):
      step()
  reset()
  graph.replay()            # warm-up
  reset()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  torch.cuda.synchronize()
  e0.record()
  graph.replay()
  e1.record()
  torch.cuda.synchronize()
  ms = e0.elapsed_time(e1)
  reset()
  fired = 0
  for _ in range(K):          # the same K steps again, counting
    step()
    fired += int(spikes.sum().item())
  return {'value': fired * DEGREE / (ms * 1e-3), 'unit': UNIT, 'ms_per_step': ms / K, 'spikes_per_step': fired / K,
          'gpu_launches_per_step': 2,
          'what': 'lif_exp_step_float (conductance decay + LIF update + threshold + spike compaction, 1e6 neurons) then '
                  'event_cbcsr_matvec_list_heter_float on the prepared matrix (fixed-point accumulation), K steps in one '
                  'CUDA graph; compare prepared_fixed_point.ms_per_step (spike scan + scatter, no neuron update)'}


def reference_cuda_c3(torch, work, ev_dev, shape, first, count, ops_per_step):
  """The reference's own CUDA kernel (lib/gpu_event_csr_matvec.cu:74-95 behind its wrapper :148-217, recompiled
  for sm_100a) on the same matrix and spikes, same GPU, outside every timed region of this library."""
  import ctypes
  from oracle import ref
  from brainpylib_b200 import gpu_ops
  if not ref.available_gpu():
    return {'unavailable': 'oracle/_ref/libref_gpu.so is not built on this machine'}
  y_ref = torch.empty(shape[1], dtype=torch.float32, device=ev_dev.device)
  opaque = gpu_ops.build_twouint_onebool_descriptor(shape[0], shape[1], True)
  fn = ref.gpu_fn('event_csr_matvec_heter_float_float')
  default = torch.cuda.default_stream(ev_dev.device)

  def call(s):
    bufs = (ctypes.c_void_p * 5)(work['data'].data_ptr(), work['indices'].data_ptr(), work['indptr'].data_ptr(),
                                 ev_dev[s].data_ptr(), y_ref.data_ptr())
    fn(None, bufs, opaque, len(opaque))   # legacy default stream: its cudaMemset and its kernel are ordered there
  torch.cuda.synchronize()
  call(first)
  torch.cuda.synchronize()
  a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  a.record(default)
  for s in range(first, first + count):
    call(s)
  b.record(default)
  torch.cuda.synchronize()
  ms = a.elapsed_time(b)
  return {'value': sum(ops_per_step[first:first + count]) / (ms * 1e-3), 'unit': UNIT, 'ms_per_step': ms / count,
          'steps': count, 'kernel': 'lib/gpu_event_csr_matvec.cu event_csr_matvec_heter_float_float (one warp per row, '
          'one atomicAdd per synapse), host-launched back to back, CUDA events on the legacy default stream'}


def run_e2e_single(torch, work, ev_host, shape, W, K, device, cb):
  """End to end with HOST buffers through the library's public call for it (brainpylib_b200.HostSteps ->
  bpl_run_host_steps -> the custom-call target on the prepared matrix): every step copies that step's spike vector
  from pinned host memory to the device, runs the target and copies the result back to pinned host memory.  Three
  streams (copy in, compute, copy out) over rings of three buffers, enqueued by native code; time = CUDA events
  around the whole run."""
  import brainpylib_b200 as bpl
  from brainpylib_b200 import event_ops
  runner = bpl.HostSteps(cb, shape=shape, events_dtype=torch.float32)
  y_host = torch.empty((3, shape[1]), dtype=torch.float32).pin_memory()
  runner.run(ev_host[:max(W, 1)], y_host)
  y_host.fill_(0.0)
  ms = runner.run(ev_host[W:W + K], y_host)
  last = y_host[(K - 1) % 3]
  if not torch.isfinite(last).all() or float(last.abs().sum()) == 0.0:
    raise SystemExit('e2e: the result copied back to the host is empty')
  want = event_ops.event_cbcsr_matvec_raw(cb, ev_host[W + K - 1].to(device))
  if not torch.allclose(last.to(device), want, rtol=1e-5, atol=1e-2):
    raise SystemExit('e2e: the result copied back to the host differs from the operator result')
  return {'ms': ms, 'h2d': 4 * shape[0], 'd2h': 4 * shape[1]}


def run_sharded(args, torch, dist, device, world):
  """N > 1: shards by post-synaptic range, one launch per step (push of the next step's spike list to every peer
  fused with this step's scatter).  Headline: the shard prepared into the column-blocked layout (float accumulation);
  the same step on the plain CSR shard is timed beside it."""
  from brainpylib_b200 import _lib, event_ops, gpu_ops, sharded
  rank = dist.get_rank()
  K, W = args.steps, args.warmup
  n_neurons = args.neurons
  work = build_workload(W + K, keep_host_matrix=False, device=device, shard=(rank, world), n_neurons=n_neurons)
  log(f'[bench] rank {rank}: workload built in {work["gen_seconds"]:.1f}s, '
      f'{work["indices"].numel():,} synapses on device')
  shape = work['shape']
  per = n_neurons // world
  mine = slice(rank * per, (rank + 1) * per)
  ops_per_step = [int(np.count_nonzero(e)) * DEGREE for e in work['events']]
  total_ops = sum(ops_per_step[W:W + K])
  ev_all = np.stack(work['events'])
  ev_host_mine = torch.from_numpy(np.ascontiguousarray(ev_all[:, mine])).pin_memory()   # this rank's own spike sources
  ev_dev_mine = ev_host_mine.to(device)
  ev_dev_full = torch.from_numpy(ev_all[W + K - 1]).to(device)                          # last step, for the check
  lib = _lib.lib()
  peak, peak_src = measured_peaks()
  exchange = sharded.PushExchange(n_neurons, dtype=torch.float32, device=device, slots=4)
  n_y = 3
  y_ring = [torch.empty(shape[1], dtype=torch.float32, device=device) for _ in range(n_y)]
  t0 = time.perf_counter()
  prepared = event_ops.csr_to_column_blocked(work['data'], work['indices'], work['indptr'], shape=shape,
                                             block_width=event_ops.default_block_width(shape[1], device, reserve=4))
  torch.cuda.synchronize()
  prepare_ms = (time.perf_counter() - t0) * 1e3

  def run_steps(first, count, layout):
    exchange.prime(ev_dev_mine[first], y_ring[0])
    for i in range(count):
      last = i == count - 1
      y_next, ev_next = (None, None) if last else (y_ring[(i + 1) % n_y], ev_dev_mine[first + i + 1])
      if layout == 'prepared':
        exchange.step_prepared(prepared, y_ring[i % n_y], y_next, ev_next)
      else:
        exchange.step(work['data'], work['indices'], work['indptr'], y_ring[i % n_y], y_next, ev_next)

  sampler = ClockSampler(device.index)
  side = torch.cuda.Stream(device)
  graphs = []
  want = event_ops.event_csr_matvec_raw(work['data'], work['indices'], work['indptr'], ev_dev_full, shape=shape,
                                        transpose=True)

  def timed_run(layout):
    """K steps captured in one graph, CUDA events on every rank between barriers, maximum over ranks; the last
    step checked against the stand-alone operator on the assembled spike vector."""
    with torch.cuda.stream(side):
      run_steps(0, min(max(W, 3), W + K), layout)
    torch.cuda.synchronize()
    dist.barrier()
    graph, warm = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
      run_steps(W, K, layout)
    with torch.cuda.graph(warm, stream=side):
      run_steps(0, max(W, 1), layout)
    graphs.extend((graph, warm))
    warm.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    exchange.check_all(dist)
    y_last = y_ring[(K - 1) % n_y].clone()
    torch.cuda.synchronize()
    if not torch.allclose(y_last, want, rtol=1e-5, atol=1e-2):
      raise SystemExit(f'sharded step ({layout}): the result of the last step differs from the stand-alone operator')
    return t.item()

  layout = sharded.preferred_layout(shape[1])        # the storage of the shard the library recommends at this size
  other = 'csr' if layout == 'prepared' else 'prepared'
  shard = {'prepared': prepared, 'csr': (work['data'], work['indices'], work['indptr'])}
  with sampler:
    ms_by_layout = {'csr': timed_run('csr'), 'prepared': timed_run('prepared')}
    ms = ms_by_layout[layout]
    # the scatter of this rank's shard alone (stand-alone operators on the assembled vector), for the roofline
    name = 'event_csr_matvec_heter_float_float'
    opaque = gpu_ops.build_twouint_onebool_descriptor(shape[0], shape[1], True)
    ws = torch.empty(_lib.workspace_bytes(name, opaque), dtype=torch.uint8, device=device)
    ev_rot = [torch.from_numpy(ev_all[W + i]).to(device) for i in range(min(K, 8))]
    y_tmp = torch.empty(shape[1], dtype=torch.float32, device=device)
    cb_name = 'event_cbcsr_matvec_heter_float_float'
    cb_opaque = event_ops._cb_descriptor(shape[0], shape[1], prepared.block_width, prepared.scale_log2,
                                         prepared.team_lanes_log2)
    cb_ws = torch.empty(_lib.workspace_bytes(cb_name, cb_opaque), dtype=torch.uint8, device=device)
    k_ms_by_layout = {
      'csr': kernel_time_ms(torch, lib, lambda s: event_ops.event_csr_matvec_raw(
        work['data'], work['indices'], work['indptr'], ev_rot[s % len(ev_rot)], shape=shape, transpose=True, out=y_tmp,
        workspace=ws), 0, min(K, 16)),
      'prepared': kernel_time_ms(torch, lib, lambda s: event_ops.event_cbcsr_matvec_raw(
        prepared, ev_rot[s % len(ev_rot)], out=y_tmp, workspace=cb_ws), 0, min(K, 16))}
    # ---- e2e: own spikes in, own slice of the result out, every step, through the exchange ----
    e2e = run_e2e_sharded(torch, dist, shard[layout], exchange, ev_host_mine, shape, W, K, device, want)
  n_act = float(np.mean([o / DEGREE for o in ops_per_step[W:W + K]]))
  s_local = float(work['indices'].numel()) / (n_neurons * DEGREE) * n_act * DEGREE   # this rank's synapses per step
  k_bytes_by_layout = {'prepared': 6.0 * s_local + 8.0 * n_act * prepared.n_blocks + 4.0 * shape[1],
                       'csr': 8.0 * s_local + 8.0 * n_act + 4.0 * shape[1]}
  kernel_name = {'prepared': 'event_cb_scatter_kernel on one rank\'s prepared shard (stand-alone)',
                 'csr': 'row_scatter_kernel<float, heter, list, vec> on one rank\'s CSR shard (stand-alone)'}
  traffic_ratio = {'prepared': 1.14, 'csr': 1.046}
  step_call = {'prepared': 'bpl_sharded_cb_step', 'csr': 'bpl_sharded_step'}
  k_bytes, k_ms = k_bytes_by_layout[layout], k_ms_by_layout[layout]
  step_bytes = k_bytes + 4.0 * per + 4.0 * shape[1] + 4.0 * n_act * world
  achieved = k_bytes / (k_ms * 1e-3) / 1e9
  line = {
    'metric': METRIC, 'value': total_ops / (ms * 1e-3), 'unit': UNIT, 'n_gpus': world, 'steps': K, 'warmup': W,
    'ms_per_step': ms / K, 'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32',
    'data': 'synthetic',
    'config': {'workload': WORKLOAD if n_neurons == N_NEURONS else f'REDUCED TWIN of C3: {n_neurons} neurons x 1000 synapses',
               'l2': 'inputs larger than L2 in total: each step streams a different part of the 8 GB matrix',
               'sharding': f'post-synaptic neurons (matrix columns) split over {world} ranks; shard layout "{layout}" '
                           f'(sharded.preferred_layout({shape[1]}): column-blocked down to 200,000 columns per rank, plain '
                           'CSR below); each rank owns 1/N of the spike sources; ONE launch per step: the kernel pushes '
                           'the compacted spikes of step s+1 into every peer over NVLink (peer stores), waits (bounded) '
                           'for the lists of step s and scatters them; no collective on the data path'},
    'e2e': {'value': total_ops / (e2e['ms'] * 1e-3), 'unit': UNIT, 'h2d_bytes_per_step': e2e['h2d'],
            'd2h_bytes_per_step': e2e['d2h'], 'ms_per_step': e2e['ms'] / K,
            'path': f'PushExchange.run_host_steps (bpl_sharded_prime, then {step_call[layout]} per step, enqueued by one '
                    'native call): per rank its own n/N spikes from pinned host memory in, its own slice of the result '
                    'out to pinned host memory, every step'},
    'gpu_launches': K + 1,     # prime once, then one kernel per step
    'roofline': {'bound': 'hbm', 'kernel': kernel_name[layout],
                 'achieved': achieved, 'peak': peak, 'unit': 'GB/s', 'frac': achieved / peak, 'peak_source': peak_src,
                 'traffic': traffic_ratio[layout] * k_bytes,
                 'traffic_source': 'ncu dram__bytes on a reduced twin, scaled by algorithmic bytes',
                 'algorithmic_bytes_per_launch': k_bytes, 'kernel_us': k_ms * 1e3,
                 'step': {'algorithmic_bytes': step_bytes, 'us': ms / K * 1e3,
                          'frac': step_bytes / (ms / K * 1e-3) / 1e9 / peak}},
    'prepared_matrix': {'bytes': prepared.nbytes(), 'block_width': prepared.block_width, 'n_blocks': prepared.n_blocks,
                        'team_lanes': 1 << prepared.team_lanes_log2, 'prepare_ms': prepare_ms},
    'other_layout': {'layout': other, 'value': total_ops / (ms_by_layout[other] * 1e-3), 'unit': UNIT,
                     'ms_per_step': ms_by_layout[other] / K,
                     'path': f'PushExchange step on the "{other}" shard ({step_call[other]}), same graph-of-K-steps timing',
                     'kernel_us': k_ms_by_layout[other] * 1e3,
                     'roofline_frac': k_bytes_by_layout[other] / (k_ms_by_layout[other] * 1e-3) / 1e9 / peak},
    'clocks': sampler.summary(),
  }
  if rank == 0:
    emit(line)
  # Tear down in a fixed order: the captured graphs must go before the communicator.  A process that still
  # cannot finish the teardown within 30 s leaves anyway: the measurement is complete and printed.
  sys.stdout.flush()
  sys.stderr.flush()
  watchdog = threading.Timer(30.0, lambda: os._exit(0))
  watchdog.daemon = True
  watchdog.start()
  torch.cuda.synchronize()
  dist.barrier()
  for g in graphs:
    g.reset()
  torch.cuda.synchronize()
  dist.destroy_process_group()
  watchdog.cancel()


def run_e2e_sharded(torch, dist, shard, exchange, ev_host_mine, shape, W, K, device, want_last):
  """End to end on N ranks through PushExchange.run_host_steps (bpl_sharded_run_host_steps): per step a rank copies
  ITS OWN n/N spikes of the next step from pinned host memory, runs the one-launch step (push to the peers + scatter
  of the current step) and copies ITS OWN slice of the result to pinned host memory, on three streams over rings of
  three buffers.  Time: CUDA events around the run on every rank, started together after a barrier, maximum over
  ranks."""
  y_host = torch.empty((3, shape[1]), dtype=torch.float32).pin_memory()

  def run(first, count):
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    ms = exchange.run_host_steps(shard, ev_host_mine[first:first + count], y_host)
    torch.cuda.synchronize()
    dist.barrier()
    return ms

  run(0, max(W, 1))
  t = torch.tensor([run(W, K)], device=device)
  dist.all_reduce(t, op=dist.ReduceOp.MAX)
  exchange.check_all(dist)
  if not torch.allclose(y_host[(K - 1) % 3].to(device), want_last, rtol=1e-5, atol=1e-2):
    raise SystemExit('e2e: the slice copied back to the host differs from the stand-alone operator result')
  return {'ms': t.item(), 'h2d': 4 * ev_host_mine.shape[1], 'd2h': 4 * shape[1]}


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument('--gpus', type=int, default=1)
  ap.add_argument('--steps', type=int, default=200)
  ap.add_argument('--warmup', type=int, default=5)
  ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
  ap.add_argument('--no-cpu-baseline', action='store_true')
  ap.add_argument('--config', default='c3', choices=['c1', 'c2', 'c3', 'c4', 'c5', 'a13'],
                  help='c3 (default) is the benchmark; the other configurations print their own JSON lines '
                       '(see bench_configs.py)')
  ap.add_argument('--one-rank-of', type=int, default=1,
                  help='profiler aid (1 GPU): run rank 0\'s shard of an N-rank job through the one-launch sharded step')
  ap.add_argument('--neurons', type=int, default=N_NEURONS,
                  help='reduced twin of the workload (multiple of 100000), for profiler captures only')
  args = ap.parse_args()
  keep_stdout_for_the_result()
  if args.warmup < 3 and args.impl == 'ours':
    log('[bench] note: fewer than 3 warm-up steps requested; the timing rules ask for >= 3')
  if args.config != 'c3':
    import bench_configs
    bench_configs.RESULT_OUT = _RESULT_OUT
    return bench_configs.main([args.config, '--warmup', str(args.warmup)])
  if args.impl == 'reference':
    run_reference(args)
  else:
    run_ours(args)


if __name__ == '__main__':
  main()
