"""Sparse operators (mirrors brainpylib/sparse_ops.py).

``csr_matvec`` keeps the signature and checks of
brainpylib/_src/sparse_ops/sparse_csr_matvec.py:26-98 and adds a keyword-only
``transpose`` (documented there, :53-55, but never implemented).  ``cusparse_csr_matvec``
keeps the signature of brainpylib/_src/sparse_ops/cusparse_matvec.py:26-96; the reference
lowers it to jaxlib's cuSPARSE, here it runs the same CUDA kernels as ``csr_matvec``.
"""
from typing import Tuple, Union

import torch

from . import _lib, gpu_ops
from ._checks import as_tensor, contiguous, device_of, float_suffix, loop_vmap

__all__ = ['csr_matvec', 'cusparse_csr_matvec', 'csr_to_coo', 'coo_to_csr', 'csr_to_dense']


def csr_matvec_raw(data, indices, indptr, vector, *, shape, transpose=False, method='vector', out=None):
  """The primitive: checked, contiguous CUDA tensors in, result out (no autograd)."""
  homo = '_homo' if data.shape[0] == 1 else '_heter'
  opaque = gpu_ops.build_double_size_descriptor(shape[0], shape[1])
  if transpose:
    name = 'csr_matvec_transpose' + homo + float_suffix(data.dtype)
  else:
    name = 'csr_matvec' + homo + '_' + method + float_suffix(data.dtype)
  if out is None:
    out = torch.empty(shape[1] if transpose else shape[0], dtype=data.dtype, device=data.device)
  buffers = [data, indices, indptr, vector, out]
  if method == 'adaptive' and not transpose:
    buffers.insert(3, None)   # the reference's row_blocks operand; unused by this library
  _lib.call(name, buffers, opaque, device=data.device)
  return out


def csr_to_coo(indices, indptr):
  """Row and column ids of every stored entry (brainpylib/_src/sparse_ops/utils.py:40-51)."""
  counts = (indptr[1:] - indptr[:-1]).to(torch.int64)
  row = torch.repeat_interleave(torch.arange(indptr.shape[0] - 1, device=indptr.device), counts)
  return row, indices.to(torch.int64)


def coo_to_csr(pre_ids, post_ids, *, num_row):
  """Sort COO entries by row and build ``(indices, indptr)``
  (intent of brainpylib/_src/sparse_ops/utils.py:21-38)."""
  order = torch.argsort(pre_ids.to(torch.int64), stable=True)
  indices = post_ids[order].to(torch.int32)
  counts = torch.bincount(pre_ids.to(torch.int64), minlength=num_row)
  indptr = torch.zeros(num_row + 1, dtype=torch.int64, device=pre_ids.device)
  indptr[1:] = torch.cumsum(counts, 0)
  return indices, indptr.to(torch.int32)


def csr_to_dense(data, indices, indptr, *, shape):
  """Dense matrix of a CSR triple; duplicate entries add (brainpylib/_src/sparse_ops/utils.py:54-82)."""
  data = torch.atleast_1d(data)
  row, col = csr_to_coo(indices, indptr)
  dense = torch.zeros(shape, dtype=data.dtype, device=indices.device)
  vals = data.expand(indices.shape[0]) if data.shape[0] == 1 else data
  dense.index_put_((row, col), vals, accumulate=True)
  return dense


class _CSRMatvec(torch.autograd.Function):
  """Differentiation and batching rules of brainpylib/_src/sparse_ops/cusparse_matvec.py:281-307.
  Reverse mode: w.r.t. the vector the same product with ``not transpose``; w.r.t. homogeneous data
  ``<ct, op(1, v)>``; w.r.t. heterogeneous data ``v[row] * ct[col]`` if transpose else ``v[col] * ct[row]``.
  Forward mode (:281-286): ``op(data_dot, v) + op(data, v_dot)``.  Batching: a loop over the batch."""

  @staticmethod
  def forward(data, indices, indptr, vector, shape, transpose, method):
    return csr_matvec_raw(data, indices, indptr, vector, shape=shape, transpose=transpose, method=method)

  @staticmethod
  def setup_context(ctx, inputs, output):
    data, indices, indptr, vector, shape, transpose, method = inputs
    ctx.save_for_backward(data, indices, indptr, vector)
    ctx.save_for_forward(data, indices, indptr, vector)
    ctx.shape, ctx.transpose, ctx.method = shape, transpose, method

  @staticmethod
  def backward(ctx, ct):
    data, indices, indptr, vector = ctx.saved_tensors
    shape, transpose = ctx.shape, ctx.transpose
    ct = contiguous(ct)
    g_data = g_vec = None
    if ctx.needs_input_grad[0]:
      if data.shape[0] == 1:
        ones = torch.ones(1, dtype=data.dtype, device=data.device)
        g_data = torch.dot(ct, _CSRMatvec.apply(ones, indices, indptr, vector, shape, transpose, 'vector')).reshape(1)
      else:
        row, col = csr_to_coo(indices, indptr)
        g_data = vector[row] * ct[col] if transpose else vector[col] * ct[row]
    if ctx.needs_input_grad[3]:
      g_vec = _CSRMatvec.apply(data, indices, indptr, ct, shape, not transpose, 'vector')
    return g_data, None, None, g_vec, None, None, None

  # (through `apply`, not the raw kernels: under torch.func transforms tangents arrive wrapped)
  @staticmethod
  def jvp(ctx, data_dot, _indices, _indptr, vector_dot, _shape, _transpose, _method):
    data, indices, indptr, vector = ctx.saved_tensors
    args = (ctx.shape, ctx.transpose, ctx.method)
    tangent = None
    if data_dot is not None:
      tangent = _CSRMatvec.apply(contiguous(data_dot), indices, indptr, vector, *args)
    if vector_dot is not None:
      t = _CSRMatvec.apply(data, indices, indptr, contiguous(vector_dot), *args)
      tangent = t if tangent is None else tangent + t
    return tangent

  @staticmethod
  def vmap(info, in_dims, data, indices, indptr, vector, shape, transpose, method):
    return loop_vmap(_CSRMatvec.apply, info, in_dims, (data, indices, indptr, vector, shape, transpose, method))


def cbcsr_matvec_raw(prepared, vector, *, transpose, out=None):
  """``y = A^T x`` (``transpose``) or ``y = A x`` on a matrix converted once with ``event_ops.csr_to_column_blocked``
  (float accumulation); targets ``cbcsr_matvec_transpose_heter_float`` / ``cbcsr_matvec_heter_float``.  No counterpart
  in the reference."""
  from . import event_ops
  n_row, n_col = prepared.shape
  n_in, n_out = (n_row, n_col) if transpose else (n_col, n_row)
  if prepared.scale_log2 is not None:
    raise ValueError('the dense-vector product needs a matrix prepared with accumulate=\'float\'')
  if vector.dtype != torch.float32 or vector.shape != (n_in,):
    raise ValueError(f'vector must be float32 of shape ({n_in},)')
  opaque = event_ops._cb_descriptor(n_row, n_col, prepared.block_width, None, prepared.team_lanes_log2)
  if out is None:
    out = torch.empty(n_out, dtype=torch.float32, device=vector.device)
  name = 'cbcsr_matvec_transpose_heter_float' if transpose else 'cbcsr_matvec_heter_float'
  _lib.call(name, [prepared.groups, prepared.offsets, vector, out], opaque, device=vector.device)
  return out


def cbcsr_matvec_transpose_raw(prepared, vector, *, out=None):
  return cbcsr_matvec_raw(prepared, vector, transpose=True, out=out)


class _CSRMatvecPrepared(torch.autograd.Function):
  """The dense-vector product on the prepared matrix, either orientation.  Linear in ``x``: reverse mode is the other
  orientation on the same prepared matrix, forward mode the same product on the tangent; the prepared weights are
  constants (no gradient w.r.t. ``data``)."""

  @staticmethod
  def forward(vector, prepared, transpose):
    return cbcsr_matvec_raw(prepared, vector, transpose=transpose)

  @staticmethod
  def setup_context(ctx, inputs, output):
    _vector, ctx.prepared, ctx.transpose = inputs

  @staticmethod
  def backward(ctx, ct):
    g_vec = None
    if ctx.needs_input_grad[0]:
      g_vec = _CSRMatvecPrepared.apply(contiguous(ct), ctx.prepared, not ctx.transpose)
    return g_vec, None, None

  @staticmethod
  def jvp(ctx, vector_dot, _prepared, _transpose):
    if vector_dot is None:
      return None
    return _CSRMatvecPrepared.apply(contiguous(vector_dot), ctx.prepared, ctx.transpose)

  @staticmethod
  def vmap(info, in_dims, vector, prepared, transpose):
    return loop_vmap(_CSRMatvecPrepared.apply, info, in_dims, (vector, prepared, transpose))


def _prepare(data, indices, indptr, vector):
  device = device_of(data, indices, indptr, vector)
  data = torch.atleast_1d(as_tensor(data, device))
  return device, data, as_tensor(indices, device), as_tensor(indptr, device), as_tensor(vector, device)


def _dispatch(data, indices, indptr, vector, shape, transpose, method):
  shape = (int(shape[0]), int(shape[1]))
  if indices.dtype not in (torch.int32, getattr(torch, 'uint32', torch.int32)):
    indices = indices.to(torch.int32)
  if indptr.dtype not in (torch.int32, getattr(torch, 'uint32', torch.int32)):
    indptr = indptr.to(torch.int32)
  data, indices, indptr, vector = map(contiguous, (data, indices, indptr, vector))
  return _CSRMatvec.apply(data, indices, indptr, vector, shape, bool(transpose), method)


def csr_matvec(
    data: Union[float, torch.Tensor],
    indices: torch.Tensor,
    indptr: torch.Tensor,
    vector: torch.Tensor,
    *,
    shape: Tuple[int, int],
    method: str = 'vector',
    transpose: bool = False,
    prepared=None
) -> torch.Tensor:
  """CSR sparse matrix product with a dense vector.

  Parameters
  ----------
  data: tensor, float
    An array of shape ``(nse,)`` or ``(1,)``.
  indices: tensor
    An array of shape ``(nse,)``.
  indptr: tensor
    An array of shape ``(shape[0] + 1,)`` and dtype ``indices.dtype``.
  vector: tensor
    An array of shape ``(shape[0] if transpose else shape[1],)`` and dtype ``data.dtype``.
  shape: tuple of int
    A length-2 tuple representing the matrix shape.
  method: str
    ``scalar``, ``vector`` or ``adaptive``: the reference's three GPU work mappings.
    They name the same kernel here; an unknown name raises ``ValueError``.
  transpose: bool
    Whether to transpose the sparse matrix before computing.
  prepared: ColumnBlockedCSR, optional
    Not in the reference.  For float32 heterogeneous weights: the same matrix converted once with
    ``event_ops.csr_to_column_blocked`` (float accumulation).  ``transpose=True`` then accumulates in shared memory
    instead of through one L2 reduction per stored entry, ``transpose=False`` gathers the vector from shared memory
    instead of through L1 / L2.  Same result up to the order of float32 additions; the weights inside ``prepared``
    are constants for differentiation.

  Returns
  -------
  y : tensor
    The array of shape ``(shape[1] if transpose else shape[0],)``.
  """
  if method not in ['scalar', 'vector', 'adaptive']:
    raise ValueError('Only support methods: scalar, vector, and adaptive. '
                     f'But we got {method}.')
  _, data, indices, indptr, vector = _prepare(data, indices, indptr, vector)
  if data.dtype not in [torch.float32, torch.float64]:
    raise TypeError(f'Only support float32 and float64. But we got {data.dtype}.')
  if data.dtype != vector.dtype:
    raise TypeError('The types of data and vector should be the same. '
                    f'But we got {data.dtype} != {vector.dtype}.')
  assert data.ndim == indices.ndim == indptr.ndim == vector.ndim == 1
  if indptr.shape[0] != shape[0] + 1:
    raise ValueError(f'shape {shape} does not match the given indptr {tuple(indptr.shape)}.')
  if vector.shape[0] != (shape[0] if transpose else shape[1]):
    raise ValueError(f'shape {shape} does not match the given vector {tuple(vector.shape)}.')
  if prepared is not None:
    if data.dtype != torch.float32 or data.shape[0] == 1:
      raise ValueError('prepared= applies to float32 heterogeneous weights')
    if tuple(prepared.shape) != (int(shape[0]), int(shape[1])):
      raise ValueError(f'the prepared matrix has shape {prepared.shape}, not {tuple(shape)}')
    return _CSRMatvecPrepared.apply(contiguous(vector), prepared, bool(transpose))
  return _dispatch(data, indices, indptr, vector, shape, transpose, method)


def cusparse_csr_matvec(
    data: Union[float, torch.Tensor],
    indices: torch.Tensor,
    indptr: torch.Tensor,
    vector: torch.Tensor,
    *,
    shape: Tuple[int, int],
    transpose: bool = False
) -> torch.Tensor:
  """Product of CSR sparse matrix and a dense vector (the op the reference's
  differentiation rules call; same arguments as ``csr_matvec`` without ``method``)."""
  _, data, indices, indptr, vector = _prepare(data, indices, indptr, vector)
  if len(shape) != 2:
    raise ValueError(f'shape should be a tuple of int denoting (n_row, n_col). Got {shape}.')
  if not (vector.ndim == data.ndim == indices.ndim == indptr.ndim == 1):
    raise ValueError('Data dimension mismatch. All must be 1D array.')
  if data.shape[0] not in [1, indices.shape[0]]:
    raise ValueError('The size of values should be 1 or be consistent with indices.'
                     f'But we got {tuple(data.shape)} != {tuple(indices.shape)}, {tuple(data.shape)} != 1.')
  if indices.dtype.is_floating_point or indices.dtype == torch.bool:
    raise ValueError('indices should be a 1D vector with integer type.')
  if indptr.dtype.is_floating_point or indptr.dtype == torch.bool:
    raise ValueError('indptr should be a 1D vector with integer type.')
  if data.dtype != vector.dtype:
    raise ValueError(f'Types of data and vector mismatch. Got {data.dtype} != {vector.dtype}.')
  if indptr.shape[0] != shape[0] + 1:
    raise ValueError(f'shape {shape} does not match the given indptr {tuple(indptr.shape)}.')
  if vector.shape[0] != (shape[0] if transpose else shape[1]):
    raise ValueError(f'shape {shape} does not match the given vector {tuple(vector.shape)}.')
  return _dispatch(data, indices, indptr, vector, shape, transpose, 'vector')
