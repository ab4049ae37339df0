"""Timing of this library's kernels beside the reference's own CUDA kernels (lib/gpu_*.cu compiled for
sm_100a into oracle/_ref/libref_gpu.so) on the benchmark shapes, same inputs, same GPU, CUDA events,
best of a few runs.  The assertions are loose floors (a regression guard); the measured ratios are
printed (run with -s to see them)."""
import ctypes

import numpy as np
import pytest
import torch

from brainpylib_b200 import gpu_ops, jitconn_ops, workloads
from oracle import ref

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref.available_gpu(), reason='oracle/_ref/libref_gpu.so not built')]


def best_us(fn, reps=3, warm=1):
  for _ in range(warm):
    fn()
  torch.cuda.synchronize()
  best = None
  for _ in range(reps):
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    fn()
    b.record()
    torch.cuda.synchronize()
    t = a.elapsed_time(b) * 1e3
    best = t if best is None else min(best, t)
  return best


def ref_launcher(name, tensors, opaque):
  bufs = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
  fn = ref.gpu_fn(name)
  return lambda: fn(None, bufs, opaque, len(opaque))


@pytest.mark.parametrize('kind,w1,w2', [('homo', 0., 0.), ('uniform', -0.1, 0.2), ('normal', 0., 0.01)])
def test_jitconn_event_matvec_million_neurons(cuda, kind, w1, w2):
  c = workloads.config_c4()
  n = c['shape'][0]
  ev = torch.as_tensor(c['events']).to(cuda)
  for odp, floor in ((True, 0.95), (False, 4.0)):
    kw = dict(kind=kind, w1=w1, w2=w2, conn_prob=c['conn_prob'], shape=c['shape'], seed=c['seed'], transpose=False,
              outdim_parallel=odp)
    ours = best_us(lambda: jitconn_ops.event_matvec_raw(ev, **kw))
    y_ref = torch.empty(n, device=cuda)
    name = f'gpu_event_matvec{"" if odp else "_atomic"}_prob_{kind}_v2_float_bool'
    theirs = best_us(ref_launcher(name, [ev, y_ref], jitconn_ops._descriptor(kind, n, n, c['seed'], c['conn_prob'], w1, w2)),
                     reps=2)
    y = jitconn_ops.event_matvec_raw(ev, **kw)
    torch.cuda.synchronize()
    if odp or kind == 'homo':
      assert torch.equal(y, y_ref)          # 1e9 generated connections, bit-identical
    else:
      torch.testing.assert_close(y, y_ref, rtol=1e-5, atol=1e-5)
    print(f'\njitconn event matvec 1e6x1e6 {kind} outdim_parallel={odp}: ours {ours:.0f} us, reference {theirs:.0f} us, '
          f'{theirs / ours:.2f}x')
    assert theirs / ours > floor


def test_jitconn_matmat_256_by_65536(cuda):
  c = workloads.config_c5()
  X = torch.as_tensor(c['matrix']).to(cuda)
  kw = dict(kind='normal', w1=c['w_mu'], w2=c['w_sigma'], conn_prob=c['conn_prob'], shape=c['shape'], seed=c['seed'])
  ours = best_us(lambda: jitconn_ops.matmat_raw(X, **kw))
  Y_ref = torch.empty(256, c['shape'][1], device=cuda)
  opaque = gpu_ops.build_matmat_jit_prob_descriptor1(256, c['shape'][0], c['shape'][1], c['seed'],
                                                     jitconn_ops._log_p(c['conn_prob']), c['w_mu'], c['w_sigma'])
  theirs = best_us(ref_launcher('gpu_matmat_prob_prob_normal_float_v1', [X, Y_ref], opaque), reps=2)
  Y = jitconn_ops.matmat_raw(X, **kw)
  torch.cuda.synchronize()
  assert torch.equal(Y, Y_ref)
  print(f'\njitconn matmat 256x65536 @ 65536^2: ours {ours:.0f} us, reference {theirs:.0f} us, {theirs / ours:.2f}x')
  assert theirs / ours > 2.0
