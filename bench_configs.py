"""Timing of the operators on the benchmark configurations other than the headline one.

    python bench_configs.py c1|c2|c4|c5 [--steps K] [--warmup W] [--variant ...]
    python bench.py --config c2            (delegates here)

One JSON line per measured variant.  K calls are captured in one CUDA graph (so the number is
the device time of the kernels, not Python dispatch) and timed with CUDA events after W warm-up
replays of a shorter graph; configurations whose inputs would fit in the 126 MB L2 rotate
several copies of the matrix between calls.  Every line also carries

  cpu_baseline    the reference's CPU code for the operator (oracle/_ref/libref_cpu.so, the reference's own
                  serial C++; where the reference has only a numba kernel or no CPU code at all, this
                  repository's CPU restatement, kind "port") timed on the host, cores stated, on a bounded
                  sample that is described in the line;
  reference_cuda  the reference's own CUDA kernel (lib/gpu_*.cu recompiled for sm_100a into
                  oracle/_ref/libref_gpu.so) on the same inputs and the same GPU, outside the timed region of
                  this library's kernel, when that library is present.

c1  event_csr_matvec 4000 x 4000, p = 0.02, homogeneous 0.6, bool events 5 %, transpose
c2  csr_matvec 1e5 x 1e5, 100 entries per row, N(0,1) weights, both orientations
c4  jitconn event matvec 1e6 x 1e6, conn_prob 1e-3, seed 42, bool events 2 %:
    homo / uniform / normal weights x outdim_parallel True / False
c5  jitconn matmat X (256 x 65536) @ M (65536 x 65536), conn_prob 0.01, N(0, 0.01), seed 7
"""
import argparse
import ctypes
import json
import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)

from brainpylib_b200 import _lib, gpu_ops, jitconn_ops, sparse_ops, event_ops, workloads  # noqa: E402

HBM_GBS_FALLBACK = 6650.0
SM_CLOCK_HZ = 1.965e9
ISSUE_PEAK = 148 * 4 * 32 * SM_CLOCK_HZ      # thread-instructions per second at the maximum SM clock
# thread-instruction budget per generated connection (RNG step, uniform conversion, float log,
# double division + ceil + conversion, event test / weight draw), counted from the reference arithmetic
INSTR_PER_CONNECTION = {'homo': 46, 'uniform': 60, 'normal': 85}


def _hbm_peak():
  path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
  try:
    return float(json.load(open(path))['hbm_gbs']), 'measured'
  except Exception:
    return HBM_GBS_FALLBACK, 'fallback'


def time_graph(fn, steps, warmup):
  """Device time per call (microseconds) of `fn(i)` for i in range(steps), captured in one CUDA graph."""
  stream = torch.cuda.Stream()
  with torch.cuda.stream(stream):
    fn(0)
  torch.cuda.synchronize()
  graph, warm = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
  with torch.cuda.graph(warm, stream=stream):
    for i in range(max(1, warmup)):
      fn(i)
  with torch.cuda.graph(graph, stream=stream):
    for i in range(steps):
      fn(i)
  warm.replay()
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  best = None
  for _ in range(3):
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    t = e0.elapsed_time(e1) * 1e3 / steps
    best = t if best is None else min(best, t)
  return best


def time_cpu(fn, budget_seconds=5.0, max_calls=50):
  """Seconds per call of a host function: one untimed call, then calls until the budget is spent."""
  fn()
  n, total = 0, 0.0
  while n < max_calls and total < budget_seconds:
    t0 = time.perf_counter()
    fn()
    total += time.perf_counter() - t0
    n += 1
  return total / n, n


def reference_cuda_us(name, tensors, opaque, reps=3):
  """Microseconds per call of the reference's own CUDA wrapper `name` (legacy default stream, where its
  cudaMemset and its kernel are ordered), best of `reps`; None when oracle/_ref/libref_gpu.so is absent."""
  from oracle import ref
  if not ref.available_gpu():
    return None
  bufs = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
  fn = ref.gpu_fn(name)
  torch.cuda.synchronize()
  fn(None, bufs, opaque, len(opaque))
  torch.cuda.synchronize()
  best = None
  for _ in range(reps):
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(torch.cuda.default_stream())
    fn(None, bufs, opaque, len(opaque))
    b.record(torch.cuda.default_stream())
    torch.cuda.synchronize()
    t = a.elapsed_time(b) * 1e3
    best = t if best is None else min(best, t)
  return best


def ref_cuda_entry(us, what, ours_us):
  if us is None:
    return {'unavailable': 'oracle/_ref/libref_gpu.so is not built on this machine'}
  return {'us_per_call': us, 'kernel': what, 'speedup_of_this_library': us / ours_us,
          'timing': 'CUDA events around the reference wrapper on the legacy default stream, best of 3'}


RESULT_OUT = None        # bench.py sets this to the stream that takes the JSON lines (default: stdout)


def emit(**kw):
  if int(os.environ.get('RANK', '0')) == 0:     # replicas (every configuration but c5) report once
    out = RESULT_OUT if RESULT_OUT is not None else sys.stdout
    out.write(json.dumps(kw) + '\n')
    out.flush()


def bench_c1(args, device):
  c = workloads.config_c1()
  t = {k: torch.as_tensor(c[k]).to(device) for k in ('data', 'indices', 'indptr', 'events')}
  y = torch.empty(4000, device=device)
  name = 'event_csr_matvec_homo_float_bool'
  opaque = gpu_ops.build_twouint_onebool_descriptor(4000, 4000, True)
  ws = torch.empty(_lib.workspace_bytes(name, opaque), dtype=torch.uint8, device=device)
  us = time_graph(lambda i: event_ops.event_csr_matvec_raw(t['data'], t['indices'], t['indptr'], t['events'],
                                                           shape=c['shape'], transpose=True, out=y, workspace=ws),
                  args.steps, args.warmup)
  syn = int((np.diff(c['indptr'])[c['events']]).sum())
  from oracle import cpu as oracle_cpu, ref
  if ref.available_cpu():
    sec, n = time_cpu(lambda: ref.csr_event_sum(c['events'], c['indices'], c['indptr'], c['data'], 4000), 2.0, 2000)
    kind, what = 'reference', 'lib/cpu_event_sum.cc cpu_csr_event_sum_homo_f32_i32 (serial C++)'
  else:
    sec, n = time_cpu(lambda: oracle_cpu.event_csr_matvec(c['data'], c['indices'], c['indptr'], c['events'],
                                                          shape=c['shape'], transpose=True), 2.0, 2000)
    kind, what = 'port', 'CPU restatement of lib/cpu_event_sum.cc (oracle/synaptic_oracle.c)'
  y_ref = torch.empty(4000, device=device)
  ref_us = reference_cuda_us(name, [t['data'], t['indices'], t['indptr'], t['events'], y_ref], opaque)
  peak, src = _hbm_peak()
  nbytes = 4000 * 1 + 8 * int(c['events'].sum()) + 4 * syn + 8 * 4000
  emit(config='c1', metric='synaptic_ops_per_sec', value=syn / (us * 1e-6), unit='SyOp/s', us_per_call=us,
       synaptic_ops_per_call=syn, gpu_launches_per_call=2,
       note='launch-latency bound: two back-to-back kernels on ~100 KB of data',
       roofline={'bound': 'launch latency (hbm nominally)', 'achieved': nbytes / (us * 1e-6) / 1e9, 'peak': peak,
                 'unit': 'GB/s', 'frac': nbytes / (us * 1e-6) / 1e9 / peak, 'peak_source': src, 'algorithmic_bytes': nbytes},
       cpu_baseline={'value': syn / sec, 'unit': 'SyOp/s', 'cores': 1, 'kind': kind, 'sample': f'{n} calls of {what} on the same inputs',
                     'us_per_call': sec * 1e6, 'host_cores_available': os.cpu_count()},
       reference_cuda=ref_cuda_entry(ref_us, 'lib/gpu_event_csr_matvec.cu event_csr_matvec_homo_float_bool', us))


def bench_c2(args, device):
  c = workloads.config_c2()
  n, nnz = c['shape'][0], c['data'].shape[0]
  base = {k: torch.as_tensor(c[k]).to(device) for k in ('data', 'indices', 'indptr', 'vector')}
  copies = [(base['data'].clone(), base['indices'].clone()) for _ in range(4)]   # 4 x 80 MB > L2
  peak, src = _hbm_peak()
  y = torch.empty(n, device=device)
  from oracle import cpu as oracle_cpu
  for transpose in (False, True):
    def call(i):
      d, ix = copies[i % 4]
      sparse_ops.csr_matvec_raw(d, ix, base['indptr'], base['vector'], shape=c['shape'], transpose=transpose, out=y)
    us = time_graph(call, args.steps, args.warmup)
    # parity at the measured size, outside the timed region
    want = oracle_cpu.csr_matvec(c['data'], c['indices'], c['indptr'], c['vector'], shape=c['shape'], transpose=transpose)
    call(0)
    torch.cuda.synchronize()
    err = float(np.abs(y.cpu().numpy() - want).max())
    if not err < 1e-2:
      raise SystemExit(f'c2 transpose={transpose}: result differs from the CPU oracle by {err}')
    sec, ncalls = time_cpu(lambda: oracle_cpu.csr_matvec(c['data'], c['indices'], c['indptr'], c['vector'],
                                                         shape=c['shape'], transpose=transpose), 3.0, 100)
    ref_entry = {'unavailable': 'the reference computes the transposed product with jaxlib cuSPARSE, which is not installed'}
    if not transpose:
      ref_us = reference_cuda_us('csr_matvec_heter_vector_float', [base['data'], base['indices'], base['indptr'],
                                                                  base['vector'], torch.empty(n, device=device)],
                                 gpu_ops.build_double_size_descriptor(n, n))
      ref_entry = ref_cuda_entry(ref_us, 'lib/gpu_csr_matvec.cu csr_matvec_heter_vector_float (matrix L2-resident: '
                                 'the same 80 MB every call)', us)
    nbytes = 8 * nnz + 4 * (n + 1) + 4 * n + 4 * n + (4 * n if transpose else 0)
    emit(config='c2', transpose=transpose, metric='synaptic_ops_per_sec', value=nnz / (us * 1e-6), unit='SyOp/s',
         us_per_call=us, l2='4 rotating copies of the 80 MB matrix', max_abs_error_vs_cpu_oracle=err,
         roofline={'bound': 'hbm', 'achieved': nbytes / (us * 1e-6) / 1e9, 'peak': peak, 'unit': 'GB/s',
                   'frac': nbytes / (us * 1e-6) / 1e9 / peak, 'peak_source': src, 'algorithmic_bytes': nbytes},
         cpu_baseline={'value': nnz / sec, 'unit': 'SyOp/s', 'cores': 1, 'kind': 'port',
                       'sample': f'{ncalls} calls on the full matrix of the serial C restatement (oracle/synaptic_oracle.c) of the '
                                 "reference's numba kernel (sparse_csr_matvec.py:108-126 / cusparse_matvec.py:195-212; the "
                                 'reference has no compiled CPU code for this operator and numba needs the reference tree)',
                       'us_per_call': sec * 1e6, 'host_cores_available': os.cpu_count()},
         reference_cuda=ref_entry)
  # both products on the matrix prepared once into the column-blocked layout (4 prepared copies rotate)
  prepared = [event_ops.csr_to_column_blocked(d, ix, base['indptr'], shape=c['shape']) for d, ix in copies]
  for transpose in (False, True):
    def call_prepared(i):
      sparse_ops.cbcsr_matvec_raw(prepared[i % 4], base['vector'], transpose=transpose, out=y)
    us = time_graph(call_prepared, args.steps, args.warmup)
    want = oracle_cpu.csr_matvec(c['data'], c['indices'], c['indptr'], c['vector'], shape=c['shape'], transpose=transpose)
    call_prepared(0)
    torch.cuda.synchronize()
    err = float(np.abs(y.cpu().numpy() - want).max())
    if not err < 1e-2:
      raise SystemExit(f'c2 transpose={transpose} on the prepared matrix: result differs from the CPU oracle by {err}')
    nbytes = 6 * nnz + 8 * n * prepared[0].n_blocks + 4 * n + 4 * n + 4 * n
    emit(config=f'c2 on the prepared matrix (csr_matvec(..., transpose={transpose}, prepared=P))', transpose=transpose,
         metric='synaptic_ops_per_sec', value=nnz / (us * 1e-6), unit='SyOp/s', us_per_call=us,
         l2='4 rotating copies of the prepared matrix', max_abs_error_vs_cpu_oracle=err,
         prepared_matrix={'bytes': prepared[0].nbytes(), 'block_width': prepared[0].block_width,
                          'n_blocks': prepared[0].n_blocks},
         roofline={'bound': 'hbm', 'achieved': nbytes / (us * 1e-6) / 1e9, 'peak': peak, 'unit': 'GB/s',
                   'frac': nbytes / (us * 1e-6) / 1e9 / peak, 'peak_source': src, 'algorithmic_bytes': nbytes})
  del prepared
  ev = torch.as_tensor(np.random.default_rng(1).random(n) < 0.05).to(device)

  def call_ev(i):
    d, ix = copies[i % 4]
    event_ops.event_csr_matvec_raw(d, ix, base['indptr'], ev, shape=c['shape'], transpose=False, out=y)
  us = time_graph(call_ev, args.steps, args.warmup)
  nbytes = 8 * nnz + 4 * (n + 1) + n + 4 * n
  emit(config='c2-matrix event_csr_matvec transpose=False (gather over the whole matrix)', metric='stored_synapses_per_sec',
       value=nnz / (us * 1e-6), unit='synapse/s', us_per_call=us,
       roofline={'bound': 'hbm', 'achieved': nbytes / (us * 1e-6) / 1e9, 'peak': peak, 'unit': 'GB/s',
                 'frac': nbytes / (us * 1e-6) / 1e9 / peak, 'peak_source': src, 'algorithmic_bytes': nbytes})


def bench_c4(args, device):
  c = workloads.config_c4()
  n = c['shape'][0]
  n_row = args.rows or n        # fewer output rows = a shorter launch of the same kernel (profiler captures)
  ev_np = c['events']
  ev = torch.as_tensor(ev_np).to(device)
  y = torch.empty(n_row, device=device)
  variants = {'homo': (0., 0.), 'uniform': (c['uniform']['w_low'], c['uniform']['w_high'] - c['uniform']['w_low']),
              'normal': (c['normal']['w_mu'], c['normal']['w_sigma'])}
  n_fire = int(ev_np.sum())
  for kind, (w1, w2) in variants.items():
    if args.variant and kind != args.variant:
      continue
    for odp in (True, False):
      if args.odp is not None and bool(args.odp) != odp:
        continue
      kw = dict(kind=kind, w1=w1, w2=w2, conn_prob=c['conn_prob'], shape=(n_row, n), seed=c['seed'],
                transpose=False, outdim_parallel=odp, out=y)
      us = time_graph(lambda i: jitconn_ops.event_matvec_raw(ev, **kw), args.steps, args.warmup)
      # generated connections: every row walks its stream (odp) / only firing columns walk theirs
      generated = c['conn_prob'] * (n_row * n if odp else n_row * n_fire)
      rate = generated / (us * 1e-6)
      # CPU baseline: the reference's serial C++ (one std::mt19937 stream: a different matrix, timing only) on the
      # first 50,000 output rows; it walks every row (odp) or every column (not odp) of that slab
      from oracle import ref
      cpu_entry = {'unavailable': 'oracle/_ref/libref_cpu.so is not built on this machine'}
      if ref.available_cpu():
        rows_cpu = 50_000
        cw1, cw2 = (w1, w1 + w2) if kind == 'uniform' else (w1, w2)
        sec, ncalls = time_cpu(lambda: ref.cpu_jitconn_event_matvec(ev_np, kind=kind, w1=cw1, w2=cw2, conn_prob=c['conn_prob'],
                                                                    n_row=rows_cpu, n_col=n, seed=c['seed'],
                                                                    outdim_parallel=odp), 3.0, 5)
        cpu_entry = {'value': c['conn_prob'] * rows_cpu * n / sec, 'unit': 'conn/s', 'cores': 1, 'kind': 'reference',
                     'sample': f'{ncalls} calls of lib/cpu_jitconn_event_matvec{"" if odp else "_atomic"}.cpp on the first '
                               f'{rows_cpu} output rows (5e7 generated connections per call; the CPU code walks all of them in '
                               'both modes)', 'seconds_per_call': sec, 'host_cores_available': os.cpu_count()}
      ref_us = None
      if n_row == n:
        y_ref = torch.empty(n_row, device=device)
        ref_us = reference_cuda_us(f'gpu_event_matvec{"" if odp else "_atomic"}_prob_{kind}_v2_float_bool', [ev, y_ref],
                                   jitconn_ops._descriptor(kind, n_row, n, c['seed'], c['conn_prob'], w1, w2), reps=2)
      emit(config='c4', weights=kind, outdim_parallel=odp, metric='generated_connections_per_sec', value=rate,
           unit='conn/s', us_per_call=us, generated_connections=generated,
           effective_synaptic_ops=c['conn_prob'] * n_row * n_fire, rows=n_row, cpu_baseline=cpu_entry,
           reference_cuda=ref_cuda_entry(ref_us, f'lib/gpu_jitconn_event_matvec{"" if odp else "_atomic"}.cu (walks every '
                                         'stream, firing or not)', us) if n_row == n else {'skipped': 'reduced rows'},
           roofline={'bound': 'alu-issue', 'achieved': rate * INSTR_PER_CONNECTION[kind], 'peak': ISSUE_PEAK,
                     'unit': 'thread-instr/s', 'frac': rate * INSTR_PER_CONNECTION[kind] / ISSUE_PEAK,
                     'instr_per_connection_budget': INSTR_PER_CONNECTION[kind]})


def bench_c5(args, device):
  """Under torchrun every rank computes its own range of output columns (no exchange: each column has its
  own random stream); the time is the maximum over ranks, the value the whole product."""
  import torch.distributed as dist
  from brainpylib_b200 import sharded
  world, rank = int(os.environ.get('WORLD_SIZE', '1')), int(os.environ.get('RANK', '0'))
  if world > 1 and not dist.is_initialized():
    dist.init_process_group('nccl', device_id=device)
  c = workloads.config_c5(n=args.cols) if args.cols else workloads.config_c5()
  X = torch.as_tensor(c['matrix']).to(device)
  m, k = X.shape
  n = c['shape'][1]
  lo, hi = sharded.column_range(n, rank, world)
  Y = torch.empty(m, hi - lo, device=device)
  kw = dict(kind='normal', w1=c['w_mu'], w2=c['w_sigma'], conn_prob=c['conn_prob'], shape=c['shape'], seed=c['seed'],
            rank=rank, world=world, out=Y)
  if world > 1:
    dist.barrier()
  us = time_graph(lambda i: sharded.matmat_column_shard(X, **kw), args.steps, args.warmup)
  if world > 1:
    t = torch.tensor([us], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    us = t.item()
  conn = c['conn_prob'] * k * n
  macs = conn * m
  peak = world * 148 * 128 * 2 * SM_CLOCK_HZ
  if rank == 0:
    # CPU baseline: the reference has no CPU code for this operator; the serial restatement of its per-row loop
    # (lib/cpu_jitconn_matvec.cpp:61-85 applied to every row of X) on the first 1024 output columns
    from oracle import cpu as oracle_cpu
    cols_cpu = min(1024, n)
    sec, ncalls = time_cpu(lambda: oracle_cpu.jitconn_matmat(c['matrix'], kind=oracle_cpu.W_NORMAL, w1=c['w_mu'], w2=c['w_sigma'],
                                                             conn_prob=c['conn_prob'], shape=(k, cols_cpu), seed=c['seed']), 3.0, 5)
    ref_entry = {'skipped': 'sharded run or reduced columns'}
    if world == 1 and not args.cols:
      Y_ref = torch.empty(m, n, device=device)
      ref_us = reference_cuda_us('gpu_matmat_prob_prob_normal_float_v1', [X, Y_ref],
                                 gpu_ops.build_matmat_jit_prob_descriptor1(m, k, n, c['seed'], jitconn_ops._log_p(c['conn_prob']),
                                                                           c['w_mu'], c['w_sigma']), reps=2)
      ref_entry = ref_cuda_entry(ref_us, 'lib/gpu_jitconn_matmat.cu gpu_matmat_prob_prob_normal_float_v1', us)
    emit(config='c5', metric='synaptic_ops_per_sec', value=macs / (us * 1e-6), unit='MAC/s', us_per_call=us,
         n_gpus=world, scaling='strong', sharding='output columns, no exchange', generated_connections=conn,
         cpu_baseline={'value': c['conn_prob'] * k * cols_cpu * m / sec, 'unit': 'MAC/s', 'cores': 1, 'kind': 'port',
                       'sample': f'{ncalls} calls of the serial CPU restatement (oracle/jitconn_oracle.cu, host build) on the first '
                                 f'{cols_cpu} output columns, all {m} rows of X', 'seconds_per_call': sec,
                       'host_cores_available': os.cpu_count()},
         reference_cuda=ref_entry,
         roofline={'bound': 'fp32-alu', 'achieved': 2 * macs / (us * 1e-6) / 1e12, 'peak': peak / 1e12,
                   'unit': 'TFLOP/s', 'frac': 2 * macs / (us * 1e-6) / peak,
                   'smem_gather_frac': 4 * macs / (us * 1e-6) / (world * 148 * 128 * SM_CLOCK_HZ)})
  if world > 1:
    dist.destroy_process_group()


def bench_a13(args, device):
  """The legacy scatter targets (compat operators) on C2's connectivity (1e5 x 1e5, 100 per row, 1e7 connections)
  with 5 % of the pre-synaptic neurons firing, beside the reference's CUDA wrappers of the same names."""
  c = workloads.config_c2()
  n, nnz = c['shape'][0], c['data'].shape[0]
  rng = np.random.default_rng(13)
  events = torch.as_tensor(rng.random(n) < 0.05).to(device)
  data, indices, indptr = (torch.as_tensor(c[k]).to(device) for k in ('data', 'indices', 'indptr'))
  pre_ids = torch.repeat_interleave(torch.arange(n, dtype=torch.int32, device=device),
                                    (indptr[1:] - indptr[:-1]).to(torch.int64))
  values_pre = torch.as_tensor(rng.standard_normal(n).astype(np.float32)).to(device)
  y, y_ref = torch.empty(n, device=device), torch.empty(n, device=device)
  peak, src = _hbm_peak()
  active = int(events.sum()) * 100
  cases = [
    ('gpu_csr_event_sum_heter_f32_i32', 'lib/gpu_event_sum.cu:50-117', [events, indices, indptr, data, y],
     gpu_ops.build_csr_event_sum_descriptor(n, n), active, 8 * active + n + 8 * n),
    ('gpu_coo_event_sum_heter_f32_i32', 'lib/gpu_event_sum.cu:140-206', [events, pre_ids, indices, data, y],
     gpu_ops.build_coo_event_sum_descriptor(nnz, n), active, 8 * nnz + 8 * active + 8 * n),
    ('gpu_coo_atomic_sum_heter_f32_i32', 'lib/gpu_atomic_sum.cu:39-97', [values_pre, pre_ids, indices, y],
     gpu_ops.build_coo_atomic_sum_descriptor(nnz, n), nnz, 12 * nnz + 8 * n),
  ]
  for name, where, bufs, opaque, ops, nbytes in cases:
    us = time_graph(lambda i: _lib.call(name, bufs, opaque, device=device), args.steps, args.warmup)
    ref_bufs = bufs[:-1] + [y_ref]
    if name.startswith('gpu_coo_atomic_sum'):      # the reference's wrapper reads the two id arrays the other way round
      ref_bufs = [values_pre, indices, pre_ids, y_ref]
    ref_us = reference_cuda_us(name, ref_bufs, opaque)
    emit(config='a13 ' + name, metric='synaptic_ops_per_sec', value=ops / (us * 1e-6), unit='SyOp/s', us_per_call=us,
         synaptic_ops_per_call=ops,
         roofline={'bound': 'L2 reductions (hbm nominally)', 'achieved': nbytes / (us * 1e-6) / 1e9, 'peak': peak,
                   'unit': 'GB/s', 'frac': nbytes / (us * 1e-6) / 1e9 / peak, 'peak_source': src,
                   'algorithmic_bytes': nbytes},
         reference_cuda=ref_cuda_entry(ref_us, where, us))


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument('config', choices=['c1', 'c2', 'c4', 'c5', 'a13'])
  ap.add_argument('--steps', type=int, default=None)
  ap.add_argument('--warmup', type=int, default=3)
  ap.add_argument('--variant', default=None, choices=[None, 'homo', 'uniform', 'normal'])
  ap.add_argument('--odp', type=int, default=None, choices=[None, 0, 1])
  ap.add_argument('--rows', type=int, default=None, help='c4: number of output rows (default 1e6)')
  ap.add_argument('--cols', type=int, default=None, help='c5: number of output columns (default 65536)')
  args = ap.parse_args(argv)
  if args.steps is None:
    args.steps = {'c1': 200, 'c2': 40, 'c4': 3, 'c5': 3, 'a13': 20}[args.config]
  if not torch.cuda.is_available():
    raise SystemExit('a CUDA device is required (no CPU fallback)')
  _lib.lib()
  if 'LOCAL_RANK' in os.environ:
    torch.cuda.set_device(int(os.environ['LOCAL_RANK']))
  device = torch.device('cuda', torch.cuda.current_device())
  {'c1': bench_c1, 'c2': bench_c2, 'c4': bench_c4, 'c5': bench_c5, 'a13': bench_a13}[args.config](args, device)


if __name__ == '__main__':
  main(sys.argv[1:])
