"""Compile the CUDA sources under ``csrc/`` into ``libbrainpylib_b200.so`` (in-tree).

Usage: ``python -m brainpylib_b200.build [--force] [--verbose]``

sm_100a only; no fast-math (the just-in-time-connectivity kernels must reproduce the
reference's float arithmetic bit for bit).  ``-Xptxas -v`` output (registers, spills,
shared memory) is written next to the library as ``ptxas_info.txt``.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
LIB = os.path.join(HERE, 'libbrainpylib_b200.so')
BUILD_DIR = os.path.join(HERE, 'csrc', 'build')
SOURCES = ['csr_kernels.cu', 'cbcsr_kernels.cu', 'cbcsr_build.cu', 'jitconn_kernels.cu', 'jitconn_matmat_versions.cu', 'jitconn_event_v1.cu', 'neuron_kernels.cu', 'scatter_kernels.cu', 'event_info_kernels.cu',
           'exchange_kernels.cu', 'host_steps.cc', 'gpu_ops.cc']
HEADERS = ['abi.h', 'common.cuh', 'spike_scan.cuh', 'row_scatter.cuh', 'cb_scatter.cuh', os.path.join('..', '..', 'include', 'brainpylib_b200.h')]
NVCC = os.environ.get('NVCC', 'nvcc')
FLAGS = ['-O3', '-std=c++17', '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo',
         '-Xcompiler', '-fPIC', '-Xptxas', '-v', '-Xcudafe', '--diag_suppress=68']


def _sources():
  return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _stale(target, deps):
  if not os.path.exists(target):
    return True
  t = os.path.getmtime(target)
  return any(os.path.getmtime(d) > t for d in deps)


def _compile(src, verbose):
  obj = os.path.join(BUILD_DIR, os.path.splitext(src)[0] + '.o')
  deps = [os.path.join(CSRC, src)] + [os.path.join(CSRC, h) for h in HEADERS] + [os.path.abspath(__file__)]
  if not _stale(obj, deps):
    return obj, ''
  cmd = [NVCC] + FLAGS + ['-c', os.path.join(CSRC, src), '-o', obj]
  if verbose:
    print(' '.join(cmd), flush=True)
  p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
  if p.returncode != 0:
    raise RuntimeError(f'nvcc failed on {src}:\n{p.stdout}')
  return obj, p.stdout


def build(force=False, verbose=False):
  """Build the shared library if any source is newer than it.  Returns its path."""
  srcs = _sources()
  all_inputs = [os.path.join(CSRC, f) for f in srcs + HEADERS] + [os.path.abspath(__file__)]
  if not force and not _stale(LIB, all_inputs):
    return LIB
  os.makedirs(BUILD_DIR, exist_ok=True)
  if force:
    for s in srcs:
      o = os.path.join(BUILD_DIR, os.path.splitext(s)[0] + '.o')
      if os.path.exists(o):
        os.remove(o)
  with concurrent.futures.ThreadPoolExecutor(max_workers=len(srcs)) as ex:
    results = list(ex.map(lambda s: _compile(s, verbose), srcs))
  objs = [o for o, _ in results]
  # one log per source, replaced whenever that source is recompiled; ptxas_info.txt is their concatenation and so
  # always describes the objects the library is linked from
  for s, (_, log) in zip(srcs, results):
    if log:
      with open(os.path.join(BUILD_DIR, 'ptxas_' + os.path.splitext(s)[0] + '.txt'), 'w') as f:
        f.write(log)
  with open(os.path.join(BUILD_DIR, 'ptxas_info.txt'), 'w') as out:
    for s in srcs:
      part = os.path.join(BUILD_DIR, 'ptxas_' + os.path.splitext(s)[0] + '.txt')
      if os.path.exists(part):
        out.write(open(part).read())
  if force or _stale(LIB, objs):
    cmd = [NVCC, '-shared', '-o', LIB] + objs + ['-gencode', 'arch=compute_100a,code=sm_100a']
    if verbose:
      print(' '.join(cmd), flush=True)
    subprocess.check_call(cmd)
  return LIB


if __name__ == '__main__':
  path = build(force='--force' in sys.argv, verbose='--verbose' in sys.argv or '-v' in sys.argv)
  print(path)
