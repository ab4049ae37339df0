"""Just-in-time connectivity operators (mirrors brainpylib/jitconn_ops.py).

The random matrix ``M`` (connection probability ``conn_prob``) is never stored: each
row (``outdim_parallel=True``) or column (``False``) regenerates its synapses on the GPU
from the stream ``seed + index``.  Signatures, checks and dispatch follow
brainpylib/_src/jitconn_ops/matvec.py:29-284, event_matvec.py:36-144 and
matmat.py:111-242; arrays are torch CUDA tensors.

As in the reference, ``transpose`` is consumed here by swapping the two dimensions
(matvec.py:346-347): the kernels only see ``n_row`` = output length and ``n_col`` =
input length.  The GPU kernels receive ``log(1 - conn_prob)`` rounded to float32
(matvec.py:346-349 with lib/kernel_helper_descriptor.cu:34-38).
"""
from typing import Optional, Tuple

import numpy as np
import torch

from . import _lib, gpu_ops
from ._checks import loop_vmap, as_tensor, contiguous, device_of, float_suffix
from .errors import GPUOperatorNotFound

__all__ = [
  'matvec_prob_conn_homo_weight', 'matvec_prob_conn_uniform_weight', 'matvec_prob_conn_normal_weight',
  'event_matvec_prob_conn_homo_weight', 'event_matvec_prob_conn_uniform_weight',
  'event_matvec_prob_conn_normal_weight',
  'matmat_prob_conn_uniform_weight', 'matmat_prob_conn_normal_weight',
]


def _log_p(conn_prob):
  return float(np.log((1 - conn_prob) if conn_prob < 1 else 1e-40))


def _descriptor(kind, n_row, n_col, seed, conn_prob, w1, w2):
  p = _log_p(conn_prob)
  if kind == 'homo':
    return gpu_ops.build_jitconn_prob_homo_descriptor(n_row, n_col, seed, p)
  if kind == 'uniform':
    return gpu_ops.build_jitconn_prob_uniform_descriptor(n_row, n_col, seed, p, w1, w2)
  return gpu_ops.build_jitconn_prob_normal_descriptor(n_row, n_col, seed, p, w1, w2)


def matvec_raw(vector, *, kind, w1=0., w2=0., conn_prob, shape, seed, transpose, outdim_parallel, version='v2',
               out=None):
  """Primitive ``matvec_prob_{homo,uniform,normal}``: dense input vector.
  ``w1, w2`` = ``(w_low, w_high - w_low)`` or ``(w_mu, w_sigma)``.  ``version='v1'`` passes the raw
  probability in the descriptor (matvec.py:338-343) and exists row-parallel only, as in the reference."""
  n_row, n_col = (shape[1], shape[0]) if transpose else shape
  if version == 'v1':
    if not outdim_parallel:
      raise GPUOperatorNotFound(f'gpu_matvec_atomic_prob_{kind}_v1 (the reference registers no such target either)')
    if kind == 'homo':
      opaque = gpu_ops.build_jitconn_prob_homo_descriptor(n_row, n_col, seed, conn_prob)
    elif kind == 'uniform':
      opaque = gpu_ops.build_jitconn_prob_uniform_descriptor(n_row, n_col, seed, conn_prob, w1, w2)
    else:
      opaque = gpu_ops.build_jitconn_prob_normal_descriptor(n_row, n_col, seed, conn_prob, w1, w2)
  else:
    opaque = _descriptor(kind, n_row, n_col, seed, conn_prob, w1, w2)
  name = ('gpu_matvec_prob_' if outdim_parallel else 'gpu_matvec_atomic_prob_') + kind + '_' + version + \
         float_suffix(vector.dtype)
  if out is None:
    out = torch.empty(n_row, dtype=vector.dtype, device=vector.device)
  _lib.call(name, [vector, out], opaque, device=vector.device)
  return out


def event_matvec_raw(events, *, kind, w1=0., w2=0., conn_prob, shape, seed, transpose, outdim_parallel, out=None):
  """Primitive ``event_matvec_prob_{homo,uniform,normal}``.  Output dtype: float32 for bool
  events, else the events' dtype (event_matvec.py:153-155)."""
  n_row, n_col = (shape[1], shape[0]) if transpose else shape
  if events.dtype == torch.bool:
    out_dtype, event_type = torch.float32, '_bool'
  else:
    out_dtype, event_type = events.dtype, float_suffix(events.dtype)
  opaque = _descriptor(kind, n_row, n_col, seed, conn_prob, w1, w2)
  name = ('gpu_event_matvec_prob_' if outdim_parallel else 'gpu_event_matvec_atomic_prob_') + kind + '_v2' + \
         float_suffix(out_dtype) + event_type
  if out is None:
    out = torch.empty(n_row, dtype=out_dtype, device=events.device)
  _lib.call(name, [events, out], opaque, device=events.device)
  return out


def matmat_raw(matrix, *, kind, w1, w2, conn_prob, shape, seed, out=None, version='v1', workspace=True):
  """Primitive ``matmat_prob_{uniform,normal}``: ``Y = X @ M``; target ``gpu_matmat_prob_prob_<kind>_<T>_<version>``
  as brainpylib/_src/jitconn_ops/matmat.py:443-466 builds it.  ``version='v1'`` runs the ``_v1_ws`` target (same
  bits, every column's stream generated once, lists in a workspace) unless ``workspace=False`` or a tensor to use
  as the workspace is passed."""
  m, k = matrix.shape
  opaque = gpu_ops.build_matmat_jit_prob_descriptor1(m, k, shape[1], seed, _log_p(conn_prob), w1, w2)
  name = 'gpu_matmat_prob_prob_' + kind + float_suffix(matrix.dtype) + '_' + version
  if out is None:
    out = torch.empty((m, shape[1]), dtype=matrix.dtype, device=matrix.device)
  if version == 'v1' and workspace is not False:
    name += '_ws'
    if workspace is True:
      workspace = _matmat_workspace(matrix.device, _lib.workspace_bytes(name, opaque))
    _lib.call(name, [matrix, out, workspace], opaque, device=matrix.device)
  else:
    _lib.call(name, [matrix, out], opaque, device=matrix.device)
  return out


_MATMAT_WS = {}


def _matmat_workspace(device, nbytes):
  """One scratch buffer per device, grown on demand (calls on one device are stream-ordered)."""
  ws = _MATMAT_WS.get(device)
  if ws is None or ws.numel() < nbytes:
    ws = None
    _MATMAT_WS.pop(device, None)
    ws = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
    _MATMAT_WS[device] = ws
  return ws


class _Matvec(torch.autograd.Function):
  """Linear in the vector.  Reverse mode: the cotangent goes through the same operator with ``transpose`` and
  ``outdim_parallel`` both flipped, which walks the same streams and is therefore exactly ``M^T``
  (matvec.py:393-402).  Forward mode (:371-390): the same operator on the tangent.  Batching: a loop."""

  @staticmethod
  def forward(vector, kw):
    return matvec_raw(vector, **kw)

  @staticmethod
  def setup_context(ctx, inputs, output):
    ctx.kw = inputs[1]

  @staticmethod
  def backward(ctx, ct):
    if ctx.kw.get('version', 'v2') == 'v1':
      raise NotImplementedError("version='v1' has no column-parallel kernel, hence no transpose rule; use 'v2'")
    kw = dict(ctx.kw, transpose=not ctx.kw['transpose'], outdim_parallel=not ctx.kw['outdim_parallel'])
    return _Matvec.apply(contiguous(ct), kw), None

  @staticmethod
  def jvp(ctx, vector_dot, _kw):
    return None if vector_dot is None else _Matvec.apply(contiguous(vector_dot), ctx.kw)

  @staticmethod
  def vmap(info, in_dims, vector, kw):
    return loop_vmap(_Matvec.apply, info, in_dims, (vector, kw))


class _EventMatvec(torch.autograd.Function):
  """Reverse mode: the cotangent w.r.t. (floating-point) events is the dense-vector operator with flipped
  ``transpose`` and ``outdim_parallel`` (event_matvec.py:263-273).  Forward mode (:242-260): the dense-vector
  operator on ``events_dot``.  Batching: a loop."""

  @staticmethod
  def forward(events, kw):
    return event_matvec_raw(events, **kw)

  @staticmethod
  def setup_context(ctx, inputs, output):
    ctx.kw = inputs[1]

  @staticmethod
  def backward(ctx, ct):
    kw = dict(ctx.kw, transpose=not ctx.kw['transpose'], outdim_parallel=not ctx.kw['outdim_parallel'])
    return _Matvec.apply(contiguous(ct), kw), None

  @staticmethod
  def jvp(ctx, events_dot, _kw):
    return None if events_dot is None else _Matvec.apply(contiguous(events_dot), ctx.kw)

  @staticmethod
  def vmap(info, in_dims, events, kw):
    return loop_vmap(_EventMatvec.apply, info, in_dims, (events, kw))


class _Matmat(torch.autograd.Function):
  """The reference registers batching only for the matmat primitives (matmat.py:422,477), no differentiation rule."""

  @staticmethod
  def forward(matrix, kw):
    return matmat_raw(matrix, **kw)

  @staticmethod
  def setup_context(ctx, inputs, output):
    ctx.set_materialize_grads(False)

  @staticmethod
  def backward(ctx, ct):
    raise NotImplementedError('matmat_prob_conn_* has no differentiation rule (none in the reference either)')

  @staticmethod
  def vmap(info, in_dims, matrix, kw):
    return loop_vmap(_Matmat.apply, info, in_dims, (matrix, kw))


def _check_vector(vector, shape, transpose, what):
  if vector.ndim != 1:
    raise ValueError(f'{what} should be a 1D vector.')
  if len(shape) != 2:
    raise ValueError('shape should be a length-2 tuple.')
  if transpose:
    if vector.shape[0] != shape[0]:
      raise ValueError(f'Shape mismatch, vec ({vector.shape[0]},) @ mat {shape}.')
  else:
    if vector.shape[0] != shape[1]:
      raise ValueError(f'Shape mismatch, mat {shape} @ vec ({vector.shape[0]},).')


def _seed(seed):
  if seed is None:
    seed = int(np.random.randint(0, int(1e8)))
  return int(seed)


def _matvec(vector, kind, w1, w2, conn_prob, shape, seed, transpose, outdim_parallel, version):
  vector = as_tensor(vector, device_of(vector))
  _check_vector(vector, shape, transpose, 'vector')
  assert version in ['v1', 'v2']
  if not vector.dtype.is_floating_point:
    vector = vector.to(torch.float32)
  kw = dict(kind=kind, w1=w1, w2=w2, conn_prob=conn_prob, shape=(int(shape[0]), int(shape[1])), seed=_seed(seed),
            transpose=bool(transpose), outdim_parallel=bool(outdim_parallel), version=version)
  vector = contiguous(vector)
  if version == 'v1' and torch.is_grad_enabled() and vector.requires_grad:
    raise NotImplementedError("version='v1' has no column-parallel kernel, hence no transpose rule; use 'v2'")
  return _Matvec.apply(vector, kw)


def event_matvec_v1_raw(event_ids, event_num, *, kind, w1, w2, conn_prob, n_row, n_col, seed, dtype=torch.float32,
                        out=None):
  """Primitive of the counter-based scheme: target ``gpu_event_matvec_prob_{homo,uniform,normal}_{float,double}``
  (lib/gpu_ops.cc:107-112) on the event list ``event_info`` returns.  The descriptor carries the RAW probability
  (lib/gpu_jitconn_event_matvec.cu:36: ``lfsr113_double(...) < conn_prob``)."""
  if kind == 'homo':
    opaque = gpu_ops.build_jitconn_prob_homo_descriptor(n_row, n_col, seed, conn_prob)
  elif kind == 'uniform':
    opaque = gpu_ops.build_jitconn_prob_uniform_descriptor(n_row, n_col, seed, conn_prob, w1, w2)
  else:
    opaque = gpu_ops.build_jitconn_prob_normal_descriptor(n_row, n_col, seed, conn_prob, w1, w2)
  if out is None:
    out = torch.empty(n_row, dtype=dtype, device=event_ids.device)
  num = event_num.reshape(1) if event_num.ndim == 0 else event_num
  _lib.call('gpu_event_matvec_prob_' + kind + float_suffix(dtype), [event_ids, num, out], opaque, device=event_ids.device)
  return out


def _event_matvec_v1(events, kind, w1, w2, conn_prob, shape, seed, transpose, outdim_parallel):
  """``version='v1'`` of the event products (no counterpart in the reference's Python layer, which never builds
  these target names): spike compaction with ``event_info``, then the counter-based kernel.  The matrix is a
  function of ``(seed, row, column)`` alone; ``transpose`` only swaps which dimension is the output."""
  from .event_ops import event_info
  if not outdim_parallel:
    raise ValueError("version='v1' computes one output per thread (outdim_parallel=True) only")
  if torch.is_grad_enabled() and events.requires_grad:
    raise NotImplementedError("version='v1' of the event products has no differentiation rule; use 'v2'")
  n_row, n_col = (shape[1], shape[0]) if transpose else shape
  ids, num = event_info(events)
  out_dtype = torch.float32 if events.dtype == torch.bool else events.dtype
  return event_matvec_v1_raw(ids, num, kind=kind, w1=w1, w2=w2, conn_prob=conn_prob, n_row=int(n_row), n_col=int(n_col),
                             seed=_seed(seed) & 0xFFFFFFFF, dtype=out_dtype)


def _event_matvec(events, kind, w1, w2, conn_prob, shape, seed, transpose, outdim_parallel, version='v2'):
  events = as_tensor(events, device_of(events))
  _check_vector(events, shape, transpose, 'events')
  if version not in ('v1', 'v2'):
    raise ValueError(f"version must be 'v1' or 'v2', got {version!r}")
  if version == 'v1':
    return _event_matvec_v1(contiguous(events), kind, w1, w2, conn_prob, (int(shape[0]), int(shape[1])), seed,
                            bool(transpose), bool(outdim_parallel))
  kw = dict(kind=kind, w1=w1, w2=w2, conn_prob=conn_prob, shape=(int(shape[0]), int(shape[1])), seed=_seed(seed),
            transpose=bool(transpose), outdim_parallel=bool(outdim_parallel))
  return _EventMatvec.apply(contiguous(events), kw)


def matvec_prob_conn_homo_weight(
    vector: torch.Tensor,
    weight: float,
    *,
    conn_prob: float,
    shape: Tuple[int, int],
    seed: Optional[int] = None,
    transpose: bool = False,
    outdim_parallel: bool = True,
    version: str = 'v2'
) -> torch.Tensor:
  r"""Perform :math:`y = M @ v`, where :math:`M` is just-in-time randomly generated with the
  scalar ``weight`` at each connection (``transpose=True``: :math:`y = M^T @ v`).

  ``M`` generated with ``transpose=False`` differs from the ``M^T`` generated with
  ``transpose=True`` unless the pair is ``(transpose, outdim_parallel)`` and
  ``(not transpose, not outdim_parallel)``, which walk the same random streams.

  Parameters
  ----------
  vector: tensor
    The vector.
  weight: float
    The value of the random matrix.
  conn_prob: float
    The connection probability.
  shape: tuple of int
    The matrix shape.
  seed: int
    The random number generation seed (drawn on the host when ``None``).
  transpose: bool
    Transpose the random matrix or not.
  outdim_parallel: bool
    Generate along the output dimension (one stream per output, no atomics) or along
    the input dimension (one stream per input, scattered with atomics).
  """
  r = _matvec(vector, 'homo', 0., 0., conn_prob, shape, seed, transpose, outdim_parallel, version)
  weight = as_tensor(weight, r.device, r.dtype)
  return r * weight


def matvec_prob_conn_uniform_weight(
    vector: torch.Tensor,
    *,
    w_low: float,
    w_high: float,
    conn_prob: float,
    shape: Tuple[int, int],
    seed: Optional[int] = None,
    transpose: bool = False,
    outdim_parallel: bool = True,
    version: str = 'v2'
) -> torch.Tensor:
  r"""Perform :math:`y = M @ v` with connection values drawn uniformly from
  ``[w_low, w_high)``.  See :func:`matvec_prob_conn_homo_weight` for the other arguments."""
  assert w_high > w_low
  return _matvec(vector, 'uniform', w_low, w_high - w_low, conn_prob, shape, seed, transpose, outdim_parallel,
                 version)


def matvec_prob_conn_normal_weight(
    vector: torch.Tensor,
    *,
    w_mu: float,
    w_sigma: float,
    conn_prob: float,
    shape: Tuple[int, int],
    seed: Optional[int] = None,
    transpose: bool = False,
    outdim_parallel: bool = True,
    version: str = 'v2'
) -> torch.Tensor:
  r"""Perform :math:`y = M @ v` with connection values drawn from ``N(w_mu, w_sigma)``.
  See :func:`matvec_prob_conn_homo_weight` for the other arguments."""
  return _matvec(vector, 'normal', w_mu, w_sigma, conn_prob, shape, seed, transpose, outdim_parallel, version)


def event_matvec_prob_conn_homo_weight(
    events: torch.Tensor,
    weight: float,
    *,
    conn_prob: float,
    shape: Tuple[int, int],
    seed: Optional[int] = None,
    transpose: bool = False,
    outdim_parallel: bool = True,
    version: str = 'v2',
) -> torch.Tensor:
  r"""Event-driven :math:`y = M @ \mathrm{events}` with the scalar ``weight`` at each
  connection.  ``events`` is bool or floating point (its non-zero entries are the events).
  ``version='v1'`` (not reachable from the reference's Python layer) uses the counter-based generator of
  lib/kernel_helpers_random.cuh: another random matrix, defined entry by entry by ``(seed, row, column)``."""
  r = _event_matvec(events, 'homo', 0., 0., conn_prob, shape, seed, transpose, outdim_parallel, version)
  weight = as_tensor(weight, r.device, r.dtype)
  return r * weight


def event_matvec_prob_conn_uniform_weight(
    events: torch.Tensor,
    *,
    w_low: float,
    w_high: float,
    conn_prob: float,
    shape: Tuple[int, int],
    seed: Optional[int] = None,
    transpose: bool = False,
    outdim_parallel: bool = True,
    version: str = 'v2',
) -> torch.Tensor:
  r"""Event-driven product with connection values drawn uniformly from ``[w_low, w_high)``.
  ``version``: see :func:`event_matvec_prob_conn_homo_weight`."""
  assert w_high > w_low
  return _event_matvec(events, 'uniform', w_low, w_high - w_low, conn_prob, shape, seed, transpose,
                       outdim_parallel, version)


def event_matvec_prob_conn_normal_weight(
    events: torch.Tensor,
    *,
    w_mu: float,
    w_sigma: float,
    conn_prob: float,
    shape: Tuple[int, int],
    seed: Optional[int] = None,
    transpose: bool = False,
    outdim_parallel: bool = True,
    version: str = 'v2',
) -> torch.Tensor:
  r"""Event-driven product with connection values drawn from ``N(w_mu, w_sigma)``.
  ``version``: see :func:`event_matvec_prob_conn_homo_weight`."""
  return _event_matvec(events, 'normal', w_mu, w_sigma, conn_prob, shape, seed, transpose, outdim_parallel, version)


def _matmat(matrix, kind, w1, w2, conn_prob, shape, seed, version, what):
  matrix = as_tensor(matrix, device_of(matrix))
  if matrix.ndim != 2:
    raise ValueError(what)
  if len(shape) != 2:
    raise ValueError('shape should be a length-2 tuple.')
  if matrix.shape[1] != shape[0]:
    raise ValueError(f'Shape mismatch, X {tuple(matrix.shape)} @ M ({shape},).')
  if seed is None:
    raise ValueError('Seed cannot be none.')
  # the reference registers v1 for both kinds and v2 / v3 for normal weights only (lib/gpu_ops.cc:166-174); each
  # version generates its own matrix
  if version not in (('v1', 'v2', 'v3') if kind == 'normal' else ('v1',)):
    raise ValueError(f"version must be 'v1'" + (", 'v2' or 'v3'" if kind == 'normal' else '') + f' for {kind} weights, '
                     f'got {version!r}')
  if not matrix.dtype.is_floating_point:
    matrix = matrix.to(torch.float32)
  return _Matmat.apply(contiguous(matrix), dict(kind=kind, w1=w1, w2=w2, conn_prob=conn_prob,
                                                shape=(int(shape[0]), int(shape[1])), seed=int(seed), version=version))


def matmat_prob_conn_uniform_weight(
    matrix: torch.Tensor,
    *,
    w_low: float,
    w_high: float,
    conn_prob: float,
    shape: Tuple[int, int],
    seed: Optional[int] = None,
    version: str = 'v1'
) -> torch.Tensor:
  r"""Perform :math:`Y = X @ M` with :math:`M` (``shape``) generated just in time, values
  uniform in ``[w_low, w_high)``.  Equal, row by row, to
  ``matvec_prob_conn_uniform_weight(x, ..., transpose=True, outdim_parallel=True)``."""
  assert w_high > w_low
  return _matmat(matrix, 'uniform', w_low, w_high - w_low, conn_prob, shape, seed, version,
                 'matrix should be a 2D vector.')


def matmat_prob_conn_normal_weight(
    matrix: torch.Tensor,
    *,
    w_mu: float,
    w_sigma: float,
    conn_prob: float,
    shape: Tuple[int, int],
    seed: Optional[int] = None,
    version: str = 'v1'
) -> torch.Tensor:
  r"""Perform :math:`Y = X @ M` with :math:`M` (``shape``) generated just in time, values
  from ``N(w_mu, w_sigma)``.  ``version``: 'v1' (default; one random stream per output column, equal row by row
  to ``matvec_prob_conn_normal_weight(..., transpose=True)``), 'v2' (32 streams per column) or 'v3' (streams per
  row of ``matrix``): three different random matrices, as in the reference."""
  return _matmat(matrix, 'normal', w_mu, w_sigma, conn_prob, shape, seed, version,
                 'vector should be a 2D matrix.')
