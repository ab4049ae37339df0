"""Timing of the operators on the benchmark configurations other than the headline one.

    python -m brainpylib_b200.config_bench c1|c2|c4|c5 [--steps K] [--warmup W] [--variant ...]
    python bench.py --config c2            (delegates here)

One JSON line per measured variant.  K calls are captured in one CUDA graph (so the number is
the device time of the kernels, not Python dispatch) and timed with CUDA events after W warm-up
replays of a shorter graph; configurations whose inputs would fit in the 126 MB L2 rotate
several copies of the matrix between calls.

c1  event_csr_matvec 4000 x 4000, p = 0.02, homogeneous 0.6, bool events 5 %, transpose
c2  csr_matvec 1e5 x 1e5, 100 entries per row, N(0,1) weights, both orientations
c4  jitconn event matvec 1e6 x 1e6, conn_prob 1e-3, seed 42, bool events 2 %:
    homo / uniform / normal weights x outdim_parallel True / False
c5  jitconn matmat X (256 x 65536) @ M (65536 x 65536), conn_prob 0.01, N(0, 0.01), seed 7
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

from . import _lib, gpu_ops, jitconn_ops, sparse_ops, event_ops, workloads

HBM_GBS_FALLBACK = 6650.0
SM_CLOCK_HZ = 1.965e9
ISSUE_PEAK = 148 * 4 * 32 * SM_CLOCK_HZ      # thread-instructions per second at the maximum SM clock
# thread-instruction budget per generated connection (RNG step, uniform conversion, float log,
# double division + ceil + conversion, event test / weight draw), counted from the reference arithmetic
INSTR_PER_CONNECTION = {'homo': 46, 'uniform': 60, 'normal': 85}


def _hbm_peak():
  import os
  path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'MEASURED_PEAKS.json')
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


def emit(**kw):
  if int(os.environ.get('RANK', '0')) == 0:     # replicas (every configuration but c5) report once
    print(json.dumps(kw), flush=True)


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
  emit(config='c1', metric='synaptic_ops_per_sec', value=syn / (us * 1e-6), unit='SyOp/s', us_per_call=us,
       synaptic_ops_per_call=syn, gpu_launches_per_call=2,
       note='launch-latency bound: two back-to-back kernels on ~100 KB of data')


def bench_c2(args, device):
  c = workloads.config_c2()
  n, nnz = c['shape'][0], c['data'].shape[0]
  base = {k: torch.as_tensor(c[k]).to(device) for k in ('data', 'indices', 'indptr', 'vector')}
  copies = [(base['data'].clone(), base['indices'].clone()) for _ in range(4)]   # 4 x 80 MB > L2
  peak, src = _hbm_peak()
  y = torch.empty(n, device=device)
  for transpose in (False, True):
    def call(i):
      d, ix = copies[i % 4]
      sparse_ops.csr_matvec_raw(d, ix, base['indptr'], base['vector'], shape=c['shape'], transpose=transpose, out=y)
    us = time_graph(call, args.steps, args.warmup)
    nbytes = 8 * nnz + 4 * (n + 1) + 4 * n + 4 * n + (4 * n if transpose else 0)
    emit(config='c2', transpose=transpose, metric='synaptic_ops_per_sec', value=nnz / (us * 1e-6), unit='SyOp/s',
         us_per_call=us, l2='4 rotating copies of the 80 MB matrix',
         roofline={'bound': 'hbm', 'achieved': nbytes / (us * 1e-6) / 1e9, 'peak': peak, 'unit': 'GB/s',
                   'frac': nbytes / (us * 1e-6) / 1e9 / peak, 'peak_source': src, 'algorithmic_bytes': nbytes})
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
      emit(config='c4', weights=kind, outdim_parallel=odp, metric='generated_connections_per_sec', value=rate,
           unit='conn/s', us_per_call=us, generated_connections=generated,
           effective_synaptic_ops=c['conn_prob'] * n_row * n_fire, rows=n_row,
           roofline={'bound': 'alu-issue', 'achieved': rate * INSTR_PER_CONNECTION[kind], 'peak': ISSUE_PEAK,
                     'unit': 'thread-instr/s', 'frac': rate * INSTR_PER_CONNECTION[kind] / ISSUE_PEAK,
                     'instr_per_connection_budget': INSTR_PER_CONNECTION[kind]})


def bench_c5(args, device):
  """Under torchrun every rank computes its own range of output columns (no exchange: each column has its
  own random stream); the time is the maximum over ranks, the value the whole product."""
  import torch.distributed as dist
  from . import sharded
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
    emit(config='c5', metric='synaptic_ops_per_sec', value=macs / (us * 1e-6), unit='MAC/s', us_per_call=us,
         n_gpus=world, scaling='strong', sharding='output columns, no exchange', generated_connections=conn,
         roofline={'bound': 'fp32-alu', 'achieved': 2 * macs / (us * 1e-6) / 1e12, 'peak': peak / 1e12,
                   'unit': 'TFLOP/s', 'frac': 2 * macs / (us * 1e-6) / peak,
                   'smem_gather_frac': 4 * macs / (us * 1e-6) / (world * 148 * 128 * SM_CLOCK_HZ)})
  if world > 1:
    dist.destroy_process_group()


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument('config', choices=['c1', 'c2', 'c4', 'c5'])
  ap.add_argument('--steps', type=int, default=None)
  ap.add_argument('--warmup', type=int, default=3)
  ap.add_argument('--variant', default=None, choices=[None, 'homo', 'uniform', 'normal'])
  ap.add_argument('--odp', type=int, default=None, choices=[None, 0, 1])
  ap.add_argument('--rows', type=int, default=None, help='c4: number of output rows (default 1e6)')
  ap.add_argument('--cols', type=int, default=None, help='c5: number of output columns (default 65536)')
  args = ap.parse_args(argv)
  if args.steps is None:
    args.steps = {'c1': 200, 'c2': 40, 'c4': 3, 'c5': 3}[args.config]
  if not torch.cuda.is_available():
    raise SystemExit('a CUDA device is required (no CPU fallback)')
  _lib.lib()
  if 'LOCAL_RANK' in os.environ:
    torch.cuda.set_device(int(os.environ['LOCAL_RANK']))
  device = torch.device('cuda', torch.cuda.current_device())
  {'c1': bench_c1, 'c2': bench_c2, 'c4': bench_c4, 'c5': bench_c5}[args.config](args, device)


if __name__ == '__main__':
  main(sys.argv[1:])
