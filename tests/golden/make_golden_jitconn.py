"""Generates tests/golden/jitconn_reference_gpu.npz from the REFERENCE's own CUDA kernels.

Must run on a machine with a GPU and with oracle/_ref/libref_gpu.so built (the reference's
lib/gpu_jitconn_*.cu compiled for sm_100a by oracle/Makefile):

    python tests/golden/make_golden_jitconn.py [output.npz]

For every case the inputs are rebuilt from a seed (`jitconn_cases()` below, shared with the tests),
the reference kernel registered under the case's custom-call target is run on them, and only its
OUTPUT is stored.  This pins absolute values of the cuRAND-based path, which no test of the
reference pins (its tests are relational only).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

KINDS = [('homo', 0., 0.), ('uniform', -0.1, 0.2), ('normal', 0., 0.01)]
SHAPES = [((100, 200), 0.1), ((10, 1000), 0.01), ((1000, 10), 0.4), ((2, 1000), 0.1), ((1500, 2500), 0.02)]


def jitconn_cases():
  """(name, spec) for every stored case."""
  out = []
  for si, (shape, prob) in enumerate(SHAPES):
    for kind, w1, w2 in KINDS:
      for odp in (True, False):
        for ev in ('bool', 'float'):
          out.append((f'event/{shape[0]}x{shape[1]}/{kind}/odp{int(odp)}/{ev}',
                      dict(op='event', shape=shape, prob=prob, kind=kind, w1=w1, w2=w2, odp=odp, ev=ev, seed=1234 + si)))
        out.append((f'matvec/{shape[0]}x{shape[1]}/{kind}/odp{int(odp)}',
                    dict(op='matvec', shape=shape, prob=prob, kind=kind, w1=w1, w2=w2, odp=odp, seed=99 + si)))
  for m in (5, 32):
    for kind, w1, w2 in KINDS[1:]:
      if kind == 'uniform' and m % 8:
        continue   # the reference's uniform wrapper leaves columns uncomputed unless m is a multiple of its row group
      out.append((f'matmat/m{m}/{kind}', dict(op='matmat', m=m, shape=(300, 700), prob=0.05, kind=kind, w1=w1, w2=w2,
                                              seed=7)))
  return out


def case_inputs(spec):
  """Seeded numpy inputs of a case (n_in = shape[1]: transpose=False throughout)."""
  rng = np.random.default_rng(spec['seed'])
  if spec['op'] == 'event':
    ev = rng.random(spec['shape'][1]) < 0.2
    if spec['ev'] == 'float':
      ev = ev.astype(np.float32) * (rng.random(spec['shape'][1]).astype(np.float32) + 0.5)
    return ev
  if spec['op'] == 'matvec':
    return rng.standard_normal(spec['shape'][1]).astype(np.float32)
  return rng.standard_normal((spec['m'], spec['shape'][0])).astype(np.float32)


def main():
  import torch
  from brainpylib_b200 import gpu_ops, jitconn_ops
  from oracle import ref
  assert ref.available_gpu(), 'oracle/_ref/libref_gpu.so is not built'
  dev = torch.device('cuda', 0)
  store = {}
  for name, spec in jitconn_cases():
    x = torch.as_tensor(case_inputs(spec)).to(dev)
    shape, kind, w1, w2, p, seed = spec['shape'], spec['kind'], spec['w1'], spec['w2'], spec['prob'], spec['seed']
    if spec['op'] == 'matmat':
      m = spec['m']
      pad = torch.zeros(((m + 31) // 32 + 256 // shape[1] + 3) * 32 * shape[0], device=dev)
      pad[: m * shape[0]] = x.reshape(-1)
      y = torch.full((m, shape[1]), float('nan'), device=dev)
      opaque = gpu_ops.build_matmat_jit_prob_descriptor1(m, shape[0], shape[1], seed, jitconn_ops._log_p(p), w1, w2)
      ref.gpu_call(f'gpu_matmat_prob_prob_{kind}_float_v1', [pad, y], opaque)
    else:
      y = torch.full((shape[0],), float('nan'), device=dev)
      opaque = jitconn_ops._descriptor(kind, shape[0], shape[1], seed, p, w1, w2)
      atomic = '' if spec['odp'] else '_atomic'
      if spec['op'] == 'event':
        target = f'gpu_event_matvec{atomic}_prob_{kind}_v2_float_{spec["ev"]}'
      else:
        target = f'gpu_matvec{atomic}_prob_{kind}_v2_float'
      ref.gpu_call(target, [x, y], opaque)
    assert torch.isfinite(y).all(), name
    store[name] = y.cpu().numpy()
  out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                            'jitconn_reference_gpu.npz')
  np.savez_compressed(out, **store)
  print(f'{len(store)} cases -> {out} ({os.path.getsize(out)} bytes)')


if __name__ == '__main__':
  main()
