"""ctypes access to the reference's OWN kernels compiled into ``oracle/_ref/``.
TEST INFRASTRUCTURE ONLY.

``libref_cpu.so``  lib/cpu_*.{cc,cpp}: serial C++ loops; the results oracle for
                   the stored-matrix ops and the timed CPU baseline.
``libref_gpu.so``  lib/gpu_*.cu recompiled for sm_100a: the bitwise oracle for
                   the just-in-time-connectivity ops and the kernels to beat.

The kernels are ordinary C++ functions in namespace ``brainpy_lib``; they are
looked up by their Itanium-mangled names, so the reference's pybind11 registry
modules are not needed.  The libraries are built by ``oracle/Makefile`` from the
reference sources where they lie; when they are absent (no reference tree and
no prebuilt copy) ``available_*()`` is False and callers skip.
"""
import ctypes
import os
import re
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_CPU_PATH = os.path.join(_HERE, '_ref', 'libref_cpu.so')
_GPU_PATH = os.path.join(_HERE, '_ref', 'libref_gpu.so')
REFERENCE_ROOT = os.environ.get('BRAINPYLIB_REFERENCE', '/root/reference')
_cpu = _gpu = None


def build(force=False):
  """Build ``oracle/_ref`` when the reference tree is present; otherwise keep
  whatever prebuilt libraries are there."""
  if not os.path.isdir(os.path.join(REFERENCE_ROOT, 'lib')):
    return False
  if force or not (os.path.exists(_CPU_PATH) and os.path.exists(_GPU_PATH)):
    subprocess.check_call(['make', '-C', _HERE, 'ref', f'REF={REFERENCE_ROOT}'], stdout=subprocess.DEVNULL)
  return True


def available_cpu():
  return os.path.exists(_CPU_PATH)


def available_gpu():
  return os.path.exists(_GPU_PATH)


def _mangle(name, params):
  return f'_ZN11brainpy_lib{len(name)}{name}E{params}'


def cpu_fn(name, tuple_out=False):
  """Reference CPU kernel ``brainpy_lib::<name>``: ``void(void* out, const void** in)``
  or, for the jitconn family, ``void(void** out, const void** in)``."""
  global _cpu
  if _cpu is None:
    _cpu = ctypes.CDLL(_CPU_PATH)
  fn = getattr(_cpu, _mangle(name, 'PPvPPKv' if tuple_out else 'PvPPKv'))
  fn.restype = None
  return fn


def gpu_function_name(target):
  """Name of the C++ function the reference registers under the custom-call
  target ``target`` (lib/gpu_ops.cc:28-174)."""
  m = re.fullmatch(r'gpu_event_matvec(_atomic)?_prob_(homo|uniform|normal)_v2_(\w+)', target)
  if m:
    return f'event_matvec{m.group(1) or ""}_jitconn_prob_{m.group(2)}_v2_{m.group(3)}'
  m = re.fullmatch(r'gpu_matvec(_atomic)?_prob_(homo|uniform|normal)_v2_(float|double)', target)
  if m:
    return f'matvec{m.group(1) or ""}_jitconn_prob_{m.group(2)}_v2_{m.group(3)}'
  m = re.fullmatch(r'gpu_matvec_prob_(homo|uniform|normal)_v1_(float|double)', target)
  if m:
    return f'matvec_jitconn_prob_{m.group(1)}_{m.group(2)}'
  m = re.fullmatch(r'gpu_matmat_prob_prob_(normal|uniform)_(float|double)_(v\d)', target)
  if m:
    return f'jitconn_matmat_prob_{m.group(1)}_{m.group(2)}_{m.group(3)}'
  return target


def gpu_fn(target):
  """Reference CUDA wrapper registered as ``target``:
  ``void(cudaStream_t, void** buffers, const char* opaque, size_t opaque_len)``."""
  global _gpu
  if _gpu is None:
    _gpu = ctypes.CDLL(_GPU_PATH)
  fn = getattr(_gpu, _mangle(gpu_function_name(target), 'P11CUstream_stPPvPKcm'))
  fn.restype = None
  fn.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p, ctypes.c_size_t]
  return fn


def gpu_call(target, tensors, opaque):
  """Run a reference CUDA wrapper on torch CUDA tensors (operands then outputs).

  The reference zeroes its output with ``cudaMemset`` on the legacy default
  stream while the kernel runs on the stream it is given
  (lib/gpu_event_csr_matvec.cu:170-173); it is therefore always given the
  legacy default stream (handle 0) here, where the two are ordered.
  """
  import torch
  torch.cuda.synchronize()
  bufs = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
  gpu_fn(target)(None, bufs, opaque, len(opaque))
  torch.cuda.synchronize()


def _in(*arrays):
  arr = (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
  return arr


def csr_event_sum(events, indices, indptr, values, post_num):
  """lib/cpu_event_sum.cc:6-24 (homo), :49-67 (heter); bool events, int32 ids."""
  values = np.ascontiguousarray(np.atleast_1d(values))
  suf = 'f32' if values.dtype == np.float32 else 'f64'
  homo = values.shape[0] == 1
  events = np.ascontiguousarray(events, dtype=np.bool_)
  indices = np.ascontiguousarray(indices).view(np.uint32)
  indptr = np.ascontiguousarray(indptr).view(np.uint32)
  pre = np.array([events.shape[0]], dtype=np.uint32)
  post = np.array([post_num], dtype=np.uint32)
  out = np.empty(post_num, dtype=values.dtype)
  fn = cpu_fn(f'cpu_csr_event_sum_{"homo" if homo else "heter"}_{suf}_i32')
  fn(ctypes.c_void_p(out.ctypes.data), _in(pre, post, events, indices, indptr, values))
  return out


def coo_atomic(op, values, post_ids, post_num, pre_ids=None):
  """lib/cpu_atomic_sum.cc:6-41, lib/cpu_atomic_prod.cc:6-43."""
  values = np.ascontiguousarray(np.atleast_1d(values))
  suf = 'f32' if values.dtype == np.float32 else 'f64'
  post_ids = np.ascontiguousarray(post_ids).view(np.uint32)
  n = np.array([post_ids.shape[0]], dtype=np.uint32)
  post = np.array([post_num], dtype=np.uint32)
  out = np.empty(post_num, dtype=values.dtype)
  if pre_ids is None:
    fn = cpu_fn(f'cpu_coo_atomic_{op}_homo_{suf}_i32')
    fn(ctypes.c_void_p(out.ctypes.data), _in(values, post_ids, n, post))
  else:
    pre_ids = np.ascontiguousarray(pre_ids).view(np.uint32)
    fn = cpu_fn(f'cpu_coo_atomic_{op}_heter_{suf}_i32')
    fn(ctypes.c_void_p(out.ctypes.data), _in(values, pre_ids, post_ids, n, post))
  return out


def cpu_jitconn_event_matvec(events, *, kind, w1=0., w2=0., conn_prob, n_row, n_col, seed, outdim_parallel=True):
  """lib/cpu_jitconn_event_matvec.cpp:10-91 / lib/cpu_jitconn_event_matvec_atomic.cpp:10-92.

  One sequential ``std::mt19937`` stream over all rows: a DIFFERENT matrix from
  the GPU path by design, so this is a timing baseline, never a results oracle.
  ``kind``: 'homo' | 'uniform' (w1 = w_min, w2 = w_max) | 'normal' (w1 = mu, w2 = sigma).
  """
  events = np.ascontiguousarray(events)
  ev = {np.dtype(np.bool_): 'bool', np.dtype(np.float32): 'float', np.dtype(np.float64): 'double'}[events.dtype]
  out_t = 'double' if ev == 'double' else 'float'
  out = np.empty(n_row, dtype=np.float64 if out_t == 'double' else np.float32)
  log_p = np.array([np.log((1 - conn_prob) if conn_prob < 1 else 1e-40)], dtype=np.float64)
  seed_a = np.array([seed], dtype=np.uint32)
  nr, nc = np.array([n_row], dtype=np.uint32), np.array([n_col], dtype=np.uint32)
  fn = cpu_fn(f'event_matvec{"" if outdim_parallel else "_atomic"}_prob_{kind}_{out_t}_{ev}', tuple_out=True)
  outs = (ctypes.c_void_p * 1)(out.ctypes.data)
  if kind == 'homo':
    ins = _in(events, log_p, seed_a, nr, nc)
  else:
    a, b = np.array([w1], dtype=out.dtype), np.array([w2], dtype=out.dtype)
    ins = _in(events, log_p, a, b, seed_a, nr, nc)
  fn(outs, ins)
  return out


# --- the reference's numba kernels -------------------------------------------------------------
# The modules that hold them import jax at module level and cannot be imported here; the
# `@numba.njit` function definitions are cut out of the files by AST and compiled on their own.

_NUMBA_SOURCES = {
  '_event_csr_matvec_transpose_numba_imp': 'brainpylib/_src/event_ops/event_csr_matvec.py',
  '_event_csr_matvec_numba_imp': 'brainpylib/_src/event_ops/event_csr_matvec.py',
  '_csr_matvec_numba_imp': 'brainpylib/_src/sparse_ops/sparse_csr_matvec.py',
  '_csr_matvec_transpose_numba_imp': 'brainpylib/_src/sparse_ops/cusparse_matvec.py',
}
_numba_cache = {}


def numba_kernel(name):
  """Compile the reference's ``@numba.njit`` kernel ``name`` (needs the reference tree)."""
  if name in _numba_cache:
    return _numba_cache[name]
  import ast
  import numba
  path = os.path.join(REFERENCE_ROOT, _NUMBA_SOURCES[name])
  tree = ast.parse(open(path).read())
  node = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == name)
  ns = {'numba': numba, 'np': np}
  exec(compile(ast.Module(body=[node], type_ignores=[]), path, 'exec'), ns)
  _numba_cache[name] = ns[name]
  return ns[name]


def numba_event_csr_matvec(data, indices, indptr, events, *, shape, transpose):
  data = np.ascontiguousarray(np.atleast_1d(data))
  out = np.empty(shape[1] if transpose else shape[0], dtype=data.dtype)
  fn = numba_kernel('_event_csr_matvec_transpose_numba_imp' if transpose else '_event_csr_matvec_numba_imp')
  fn(out, (data, indices, indptr, events, shape, transpose))
  return out


def numba_csr_matvec(data, indices, indptr, vector, *, shape, transpose):
  data = np.ascontiguousarray(np.atleast_1d(data))
  out = np.empty(shape[1] if transpose else shape[0], dtype=data.dtype)
  if transpose:
    numba_kernel('_csr_matvec_transpose_numba_imp')(out, (data, indices, indptr, vector, shape, transpose))
  else:
    numba_kernel('_csr_matvec_numba_imp')(out, (data, indices, indptr, vector, shape))
  return out
