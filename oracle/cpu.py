"""numpy-facing wrappers of ``liboracle.so``.  TEST INFRASTRUCTURE ONLY.

Each function mirrors one reference operator and returns a fresh numpy array.
The algorithms (and the reference file:line each follows) are in
``synaptic_oracle.c`` and ``jitconn_oracle.cu``.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, 'liboracle.so')
_lib = None

W_HOMO, W_UNIFORM, W_NORMAL = 0, 1, 2


def build(force=False):
  """Compile ``liboracle.so`` (gcc + nvcc host compilation) if it is missing."""
  if force or not os.path.exists(_LIB_PATH):
    subprocess.check_call(['make', '-C', _HERE, 'oracle'], stdout=subprocess.DEVNULL)
  return _LIB_PATH


def lib():
  global _lib
  if _lib is None:
    build()
    _lib = ctypes.CDLL(_LIB_PATH)
    for suf in ('f32', 'f64'):
      for name in ('matvec', 'event_matvec', 'matmat'):
        getattr(_lib, f'oracle_jitconn_{name}_{suf}').restype = ctypes.c_uint64
    _lib.oracle_jitconn_stream.restype = ctypes.c_uint64
    _lib.oracle_count_active_synapses.restype = ctypes.c_uint64
  return _lib


def _ptr(a):
  return ctypes.c_void_p(a.ctypes.data)


def _suffix(dtype):
  dtype = np.dtype(dtype)
  if dtype == np.float32:
    return 'f32'
  if dtype == np.float64:
    return 'f64'
  raise TypeError(f'float32 or float64 expected, got {dtype}')


def _event_kind(events):
  if events.dtype == np.bool_:
    return 0
  if events.dtype == np.float32:
    return 1
  if events.dtype == np.float64:
    return 2
  raise TypeError(f'events must be bool, float32 or float64, got {events.dtype}')


def _u32(a):
  a = np.ascontiguousarray(a)
  if a.dtype not in (np.int32, np.uint32):
    raise TypeError('index arrays must be int32 or uint32')
  return a.view(np.uint32)


def event_csr_matvec(data, indices, indptr, events, *, shape, transpose=False):
  data = np.ascontiguousarray(np.atleast_1d(data))
  suf = _suffix(data.dtype)
  indices, indptr = _u32(indices), _u32(indptr)
  events = np.ascontiguousarray(events)
  y = np.empty(shape[1] if transpose else shape[0], dtype=data.dtype)
  getattr(lib(), f'oracle_event_csr_matvec_{suf}')(
    _ptr(data), ctypes.c_int(int(data.shape[0] == 1)), _ptr(indices), _ptr(indptr),
    _ptr(events), ctypes.c_int(_event_kind(events)),
    ctypes.c_uint32(shape[0]), ctypes.c_uint32(shape[1]), ctypes.c_int(bool(transpose)), _ptr(y))
  return y


def csr_matvec(data, indices, indptr, vector, *, shape, transpose=False):
  data = np.ascontiguousarray(np.atleast_1d(data))
  suf = _suffix(data.dtype)
  vector = np.ascontiguousarray(vector, dtype=data.dtype)
  indices, indptr = _u32(indices), _u32(indptr)
  y = np.empty(shape[1] if transpose else shape[0], dtype=data.dtype)
  getattr(lib(), f'oracle_csr_matvec_{suf}')(
    _ptr(data), ctypes.c_int(int(data.shape[0] == 1)), _ptr(indices), _ptr(indptr), _ptr(vector),
    ctypes.c_uint32(shape[0]), ctypes.c_uint32(shape[1]), ctypes.c_int(bool(transpose)), _ptr(y))
  return y


def _coo_atomic(op, values, post_ids, post_num, pre_ids):
  values = np.ascontiguousarray(np.atleast_1d(values))
  suf = _suffix(values.dtype)
  homo = pre_ids is None
  post_ids = _u32(post_ids)
  pre = post_ids if homo else _u32(pre_ids)
  y = np.empty(post_num, dtype=values.dtype)
  getattr(lib(), f'oracle_coo_atomic_{op}_{suf}')(
    _ptr(values), ctypes.c_int(int(homo)), _ptr(pre), _ptr(post_ids),
    ctypes.c_uint32(post_ids.shape[0]), ctypes.c_uint32(post_num), _ptr(y))
  return y


def coo_atomic_sum(values, post_ids, post_num, pre_ids=None):
  return _coo_atomic('sum', values, post_ids, post_num, pre_ids)


def coo_atomic_prod(values, post_ids, post_num, pre_ids=None):
  return _coo_atomic('prod', values, post_ids, post_num, pre_ids)


def coo_event_sum(events, pre_ids, post_ids, post_num, values):
  values = np.ascontiguousarray(np.atleast_1d(values))
  suf = _suffix(values.dtype)
  events = np.ascontiguousarray(events, dtype=np.bool_)
  pre_ids, post_ids = _u32(pre_ids), _u32(post_ids)
  y = np.empty(post_num, dtype=values.dtype)
  getattr(lib(), f'oracle_coo_event_sum_{suf}')(
    _ptr(events), _ptr(pre_ids), _ptr(post_ids), _ptr(values), ctypes.c_int(int(values.shape[0] == 1)),
    ctypes.c_uint32(pre_ids.shape[0]), ctypes.c_uint32(post_num), _ptr(y))
  return y


def count_active_synapses(indptr, events):
  indptr = _u32(indptr)
  events = np.ascontiguousarray(events)
  return int(lib().oracle_count_active_synapses(
    _ptr(indptr), _ptr(events), ctypes.c_int(_event_kind(events)), ctypes.c_uint32(indptr.shape[0] - 1)))


def jitconn_event_matvec_v1(event_ids, event_num, *, kind, w1=0., w2=0., conn_prob, n_row, n_col, seed,
                            dtype=np.float32):
  """Counter-based event product (see ``oracle_jitconn_event_v1`` in synaptic_oracle.c).  ``conn_prob``, ``w1``,
  ``w2`` are rounded to float32 first, as the descriptor builders do."""
  ids = np.ascontiguousarray(event_ids, dtype=np.int32)
  out = np.empty(n_row, dtype=dtype)
  f32 = lambda v: float(np.float32(v))
  lib().oracle_jitconn_event_v1(_ptr(ids), ctypes.c_int32(int(event_num)), ctypes.c_uint32(seed & 0xFFFFFFFF),
                                ctypes.c_double(f32(conn_prob)), ctypes.c_int(kind), ctypes.c_double(f32(w1)),
                                ctypes.c_double(f32(w2)), ctypes.c_uint32(n_row), ctypes.c_uint32(n_col),
                                ctypes.c_int(int(np.dtype(dtype) == np.float64)), _ptr(out))
  return out


def descriptor_log_p(conn_prob):
  """``log(1 - p)`` as the GPU kernels receive it: a float64 that holds a
  float32-rounded value (brainpylib/_src/jitconn_ops/matvec.py:346-349 computes a
  Python float, lib/kernel_helper_descriptor.cu:34-38 narrows it to ``float``)."""
  return float(np.float32(np.log((1 - conn_prob) if conn_prob < 1 else 1e-40)))


def _f32round(x):
  return float(np.float32(x))


def _weights(kind, w1, w2):
  return ctypes.c_double(_f32round(w1)), ctypes.c_double(_f32round(w2))


def jitconn_matvec(vector, *, kind, w1=0., w2=0., conn_prob, shape, seed, transpose=False,
                   outdim_parallel=True, return_info=False):
  """``kind``: W_HOMO (weight 1), W_UNIFORM (w1 = w_low, w2 = w_high - w_low) or
  W_NORMAL (w1 = w_mu, w2 = w_sigma)."""
  vector = np.ascontiguousarray(vector)
  suf = _suffix(vector.dtype)
  n_row, n_col = (shape[1], shape[0]) if transpose else shape
  y = np.empty(n_row, dtype=vector.dtype)
  n_conn = ctypes.c_uint64(0)
  c1, c2 = _weights(kind, w1, w2)
  fragile = getattr(lib(), f'oracle_jitconn_matvec_{suf}')(
    _ptr(vector), ctypes.c_uint32(seed & 0xffffffff), ctypes.c_double(descriptor_log_p(conn_prob)), c1, c2,
    ctypes.c_uint32(n_row), ctypes.c_uint32(n_col), ctypes.c_int(kind), ctypes.c_int(bool(outdim_parallel)),
    _ptr(y), ctypes.byref(n_conn))
  return (y, dict(fragile=int(fragile), connections=n_conn.value)) if return_info else y


def jitconn_event_matvec(events, *, kind, w1=0., w2=0., conn_prob, shape, seed, transpose=False,
                         outdim_parallel=True, out_dtype=None, return_info=False):
  events = np.ascontiguousarray(events)
  if out_dtype is None:
    out_dtype = np.float32 if events.dtype == np.bool_ else events.dtype
  suf = _suffix(out_dtype)
  n_row, n_col = (shape[1], shape[0]) if transpose else shape
  y = np.empty(n_row, dtype=out_dtype)
  n_conn = ctypes.c_uint64(0)
  c1, c2 = _weights(kind, w1, w2)
  fragile = getattr(lib(), f'oracle_jitconn_event_matvec_{suf}')(
    _ptr(events), ctypes.c_int(_event_kind(events)), ctypes.c_uint32(seed & 0xffffffff),
    ctypes.c_double(descriptor_log_p(conn_prob)), c1, c2,
    ctypes.c_uint32(n_row), ctypes.c_uint32(n_col), ctypes.c_int(kind), ctypes.c_int(bool(outdim_parallel)),
    _ptr(y), ctypes.byref(n_conn))
  return (y, dict(fragile=int(fragile), connections=n_conn.value)) if return_info else y


def jitconn_matmat(matrix, *, kind, w1, w2, conn_prob, shape, seed, return_info=False):
  matrix = np.ascontiguousarray(matrix)
  suf = _suffix(matrix.dtype)
  m, k = matrix.shape
  assert k == shape[0]
  n = shape[1]
  y = np.empty((m, n), dtype=matrix.dtype)
  n_conn = ctypes.c_uint64(0)
  c1, c2 = _weights(kind, w1, w2)
  fragile = getattr(lib(), f'oracle_jitconn_matmat_{suf}')(
    _ptr(matrix), ctypes.c_uint32(m), ctypes.c_uint32(k), ctypes.c_uint32(n), ctypes.c_uint32(seed & 0xffffffff),
    ctypes.c_double(descriptor_log_p(conn_prob)), c1, c2, ctypes.c_int(kind), _ptr(y), ctypes.byref(n_conn))
  return (y, dict(fragile=int(fragile), connections=n_conn.value)) if return_info else y


def jitconn_stream(stream_seed, *, conn_prob, extent, kind=W_HOMO, w1=0., w2=0., cap=None):
  """Positions and weights sampled by the stream ``seed + row`` over ``extent``
  positions.  Returns ``(positions int32, weights float32, n_fragile)``."""
  log_p = descriptor_log_p(conn_prob)
  if cap is None:
    cap = lib().oracle_jitconn_stream(
      ctypes.c_uint32(stream_seed & 0xffffffff), ctypes.c_double(log_p), ctypes.c_double(0), ctypes.c_double(0),
      ctypes.c_uint32(extent), ctypes.c_int(kind), None, None, ctypes.c_uint64(0), None)
  pos = np.empty(cap, dtype=np.int32)
  w = np.empty(cap, dtype=np.float32)
  fragile = ctypes.c_uint64(0)
  c1, c2 = _weights(kind, w1, w2)
  n = lib().oracle_jitconn_stream(
    ctypes.c_uint32(stream_seed & 0xffffffff), ctypes.c_double(log_p), c1, c2,
    ctypes.c_uint32(extent), ctypes.c_int(kind), _ptr(pos), _ptr(w), ctypes.c_uint64(cap), ctypes.byref(fragile))
  n = min(int(n), cap)
  return pos[:n], w[:n], fragile.value
