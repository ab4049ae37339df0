"""Generates tests/golden/stored_matrix.npz from the REFERENCE's own CPU code.

Run where the reference tree is mounted (its location is taken from the environment variable
``BRAINPYLIB_REFERENCE``):  ``python tests/golden/make_golden.py``

For every case the inputs are rebuilt from a seed (tests/cases.py), the reference's
compiled C++ kernel (lib/cpu_event_sum.cc, lib/cpu_atomic_sum.cc, lib/cpu_atomic_prod.cc,
through oracle/_ref/libref_cpu.so) and/or its numba kernel
(brainpylib/_src/event_ops/event_csr_matvec.py:313-357,
brainpylib/_src/sparse_ops/sparse_csr_matvec.py:108-126,
brainpylib/_src/sparse_ops/cusparse_matvec.py:195-212) is run, and only the OUTPUT is
stored, keyed by the case name.  The tests rebuild the same inputs and compare the CPU
oracle (and, on a GPU, the CUDA kernels) with these outputs.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, 'tests'))

import cases  # noqa: E402
from brainpylib_b200 import workloads  # noqa: E402
from oracle import ref  # noqa: E402


def golden_cases():
  """(name, kind, kwargs) for every stored case; shared with tests/test_oracle_pin.py."""
  out = []
  for i, shape in enumerate(cases.EVENT_CSR_SHAPES):
    for homo in (None, 1.0, -1.0, 0.6):
      for transpose in (True, False):
        for ev in ('bool', 'float'):
          out.append((f'event_csr/{shape[0]}x{shape[1]}/w{homo}/T{int(transpose)}/{ev}', 'event_csr',
                      dict(shape=shape, prob=0.4, seed=100 + i, homo=homo, transpose=transpose, ev=ev, rate=0.1)))
  for i, shape in enumerate(cases.CSR_SHAPES):
    for homo in (None, 1.5):
      for transpose in (True, False):
        out.append((f'csr/{shape[0]}x{shape[1]}/w{homo}/T{int(transpose)}', 'csr',
                    dict(shape=shape, prob=0.1, seed=200 + i, homo=homo, transpose=transpose)))
  out.append(('event_csr/C1', 'c1', {}))
  # benchmark-size configurations, stored as strided samples of the output (every 49th / 499th element)
  for transpose in (False, True):
    out.append((f'csr/C2/T{int(transpose)}', 'c2', dict(transpose=transpose, stride=49)))
  for step in (0, 1):
    out.append((f'event_csr/C3_rows_0_99999/step{step}', 'c3', dict(step=step, stride=499)))
  for homo in (True, False):
    for op in ('sum', 'prod'):
      out.append((f'coo_atomic_{op}/homo{int(homo)}', 'coo_atomic', dict(op=op, homo=homo, seed=300)))
  return out


def build_inputs(kind, kw):
  if kind == 'c1':
    return workloads.config_c1()
  if kind == 'c2':
    c = workloads.config_c2()
    return dict(data=c['data'], indices=c['indices'], indptr=c['indptr'], x=c['vector'], shape=c['shape'],
                transpose=kw['transpose'])
  if kind == 'c3':
    c = workloads.config_c3_first_rows(2)
    return dict(data=c['data'], indices=c['indices'], indptr=c['indptr'], shape=c['shape'], transpose=True,
                x=c['events_masked'][kw['step']][:c['shape'][0]])
  if kind in ('event_csr', 'csr'):
    data, indices, indptr, rng = cases.csr_case(kw['shape'], kw['prob'], kw['seed'], homo=kw['homo'])
    n_in = kw['shape'][0] if kw['transpose'] else kw['shape'][1]
    if kind == 'event_csr':
      x = cases.events_like(rng, n_in, kw['rate'], np.bool_ if kw['ev'] == 'bool' else np.float32)
    else:
      x = rng.uniform(-1, 1, n_in).astype(np.float32)
    return dict(data=data, indices=indices, indptr=indptr, x=x, shape=kw['shape'], transpose=kw['transpose'])
  if kind == 'coo_atomic':
    rng = np.random.default_rng(kw['seed'])
    n_pre, n_post, n_conn = 300, 200, 5000
    pre = rng.integers(0, n_pre, n_conn, dtype=np.int32)
    post = rng.integers(0, n_post, n_conn, dtype=np.int32)
    if kw['op'] == 'prod':   # keep products in range
      values = rng.uniform(0.9, 1.1, 1 if kw['homo'] else n_pre).astype(np.float32)
    else:
      values = rng.standard_normal(1 if kw['homo'] else n_pre).astype(np.float32)
    return dict(values=values, pre=pre, post=post, post_num=n_post, homo=kw['homo'], op=kw['op'])
  raise KeyError(kind)


def reference_output(kind, inp):
  if kind == 'c1':
    y_cc = ref.csr_event_sum(inp['events'], inp['indices'], inp['indptr'], inp['data'], inp['shape'][1])
    y_nb = ref.numba_event_csr_matvec(inp['data'], inp['indices'], inp['indptr'], inp['events'],
                                      shape=inp['shape'], transpose=True)
    assert np.array_equal(y_cc.view(np.uint32), y_nb.view(np.uint32)), 'reference C++ and numba kernels disagree'
    return y_cc
  if kind == 'event_csr':
    y = ref.numba_event_csr_matvec(inp['data'], inp['indices'], inp['indptr'], inp['x'],
                                   shape=inp['shape'], transpose=inp['transpose'])
    if inp['transpose'] and inp['x'].dtype == np.bool_:
      y_cc = ref.csr_event_sum(inp['x'], inp['indices'], inp['indptr'], inp['data'], inp['shape'][1])
      assert np.array_equal(y_cc.view(np.uint32), y.view(np.uint32)), 'reference C++ and numba kernels disagree'
    return y
  if kind == 'csr':
    return ref.numba_csr_matvec(inp['data'], inp['indices'], inp['indptr'], inp['x'],
                                shape=inp['shape'], transpose=inp['transpose'])
  if kind == 'c2':
    return ref.numba_csr_matvec(inp['data'], inp['indices'], inp['indptr'], inp['x'],
                                shape=inp['shape'], transpose=inp['transpose'])
  if kind == 'c3':   # the reference's serial C++ kernel on the rows a CPU can hold; events as bool (truthiness)
    return ref.csr_event_sum(inp['x'] != 0, inp['indices'], inp['indptr'], inp['data'], inp['shape'][1])
  if kind == 'coo_atomic':
    return ref.coo_atomic(inp['op'], inp['values'], inp['post'], inp['post_num'],
                          None if inp['homo'] else inp['pre'])
  raise KeyError(kind)


def main():
  assert ref.build(), 'reference tree not found'
  store = {}
  for name, kind, kw in golden_cases():
    y = reference_output(kind, build_inputs(kind, kw))
    store[name] = y[::kw['stride']].copy() if 'stride' in kw else y
  path = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'stored_matrix.npz')
  np.savez_compressed(path, **store)
  print(f'{len(store)} cases -> {path} ({os.path.getsize(path)} bytes)')


if __name__ == '__main__':
  main()
