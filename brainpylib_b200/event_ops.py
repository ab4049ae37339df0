"""Event-driven sparse operators (mirrors brainpylib/event_ops.py).

``event_csr_matvec`` keeps the signature, argument checks and error behaviour of
brainpylib/_src/event_ops/event_csr_matvec.py:32-102; arrays are torch CUDA tensors
(the reference's are JAX arrays) and the work is done by the custom-call target
``event_csr_matvec_{homo,heter}_{float,double}_{bool,float,double}`` of the CUDA
library, chosen exactly as the reference's GPU translation chooses it (:389-417).
"""
from typing import Tuple, Union

import torch

from . import _lib, gpu_ops
from .errors import GPUOperatorNotFound
from ._checks import as_tensor, contiguous, device_of, float_suffix, is_int32_like

__all__ = ['event_csr_matvec', 'event_info']

_workspaces = {}


def _workspace(device, nbytes):
  """A per-(device, stream) scratch tensor, grown on demand.  Kernels of one stream run
  in order, so one buffer per stream is safe to reuse."""
  key = (device.index, torch.cuda.current_stream(device).cuda_stream)
  ws = _workspaces.get(key)
  if ws is None or ws.numel() < nbytes:
    ws = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
    _workspaces[key] = ws
  return ws


def _target_name(data, events):
  type_name = float_suffix(data.dtype)
  data_name = '_homo' if data.shape[0] == 1 else '_heter'
  if events.dtype == torch.bool:
    vec_type = '_bool'
  else:
    if events.dtype != data.dtype:
      raise ValueError(f'events must be bool or have the dtype of data; got {events.dtype} and {data.dtype}.')
    vec_type = type_name
  return 'event_csr_matvec' + data_name + type_name + vec_type


def event_csr_matvec_raw(data, indices, indptr, events, *, shape, transpose=False, out=None, workspace=None):
  """The primitive: checked, contiguous CUDA tensors in, result out (no autograd)."""
  name = _target_name(data, events)
  if data.device.type != 'cuda':
    raise GPUOperatorNotFound(f'{name} (operands are on {data.device}, a CUDA device is required)')
  opaque = gpu_ops.build_twouint_onebool_descriptor(shape[0], shape[1], transpose)
  n_out = shape[1] if transpose else shape[0]
  if out is None:
    out = torch.empty(n_out, dtype=data.dtype, device=data.device)
  if transpose and workspace is None:
    workspace = _workspace(data.device, _lib.workspace_bytes(name, opaque))
  _lib.call(name, [data, indices, indptr, events, out, workspace], opaque, device=data.device)
  return out


class _EventCSRMatvec(torch.autograd.Function):
  """Differentiation rules of brainpylib/_src/event_ops/event_csr_matvec.py:439-463,
  written as the vector-Jacobian product torch asks for:

  * w.r.t. ``events``: ``A^T ct`` (or ``A ct``), i.e. the dense CSR product with the
    opposite ``transpose`` (:447-451).
  * w.r.t. homogeneous ``data``: ``<ct, op(1, events)>`` (:457-459).
  * w.r.t. heterogeneous ``data``: ``events[row] * ct[col]`` if transpose else
    ``events[col] * ct[row]`` (:461-462).
  """

  @staticmethod
  def forward(ctx, data, indices, indptr, events, shape, transpose):
    ctx.save_for_backward(data, indices, indptr, events)
    ctx.shape, ctx.transpose = shape, transpose
    return event_csr_matvec_raw(data, indices, indptr, events, shape=shape, transpose=transpose)

  @staticmethod
  def backward(ctx, ct):
    from .sparse_ops import csr_matvec_raw, csr_to_coo
    data, indices, indptr, events = ctx.saved_tensors
    shape, transpose = ctx.shape, ctx.transpose
    ct = contiguous(ct)
    g_data = g_events = None
    if ctx.needs_input_grad[0]:
      if data.shape[0] == 1:
        ones = torch.ones(1, dtype=data.dtype, device=data.device)
        r = event_csr_matvec_raw(ones, indices, indptr, events, shape=shape, transpose=transpose)
        g_data = torch.dot(ct, r).reshape(1)
      else:
        row, col = csr_to_coo(indices, indptr)
        ev = events.to(data.dtype)
        g_data = ev[row] * ct[col] if transpose else ev[col] * ct[row]
    if ctx.needs_input_grad[3]:
      g_events = csr_matvec_raw(data, indices, indptr, ct, shape=shape, transpose=not transpose)
    return g_data, None, None, g_events, None, None


def event_csr_matvec(
    data: Union[float, torch.Tensor],
    indices: torch.Tensor,
    indptr: torch.Tensor,
    events: torch.Tensor,
    *,
    shape: Tuple[int, int],
    transpose: bool = False
) -> torch.Tensor:
  """Product of a sparse CSR matrix and a dense event vector.

  Parameters
  ----------
  data: tensor, float
    An array of shape ``(nse,)``, or a scalar / ``(1,)`` array for homogeneous weights.
  indices: tensor
    An array of shape ``(nse,)``, int32 (uint32 accepted).
  indptr: tensor
    An array of shape ``(shape[0] + 1,)`` and dtype ``indices.dtype``.
  events: tensor
    An array of shape ``(shape[0] if transpose else shape[1],)``; bool, or the dtype of
    ``data``.  Only the truthiness of an event is used.
  shape: tuple
    A length-2 tuple representing the matrix shape.
  transpose: bool
    Whether to transpose the sparse matrix before computing.

  Returns
  -------
  y : tensor
    The array of shape ``(shape[1] if transpose else shape[0],)``.
  """
  device = device_of(data, indices, indptr, events)
  data = torch.atleast_1d(as_tensor(data, device))
  if not data.dtype.is_floating_point:
    data = data.to(torch.float32)
  indices = as_tensor(indices, device)
  indptr = as_tensor(indptr, device)
  events = as_tensor(events, device)
  # checking
  if data.ndim == 1:
    if data.shape[0] not in [1, indices.shape[0]]:
      raise ValueError('The size of data should be 1 or be consistent with indices.'
                       f'But we got {tuple(data.shape)} != {tuple(indices.shape)}, {tuple(data.shape)} != 1.')
  else:
    raise ValueError('data should be a scalar or 1D vector. '
                     f'But we got {data.ndim}-D array.')
  if indices.ndim != 1:
    raise ValueError('indices should be a 1D vector with integer type.')
  if indptr.ndim != 1:
    raise ValueError('indptr should be a 1D vector with integer type.')
  if not is_int32_like(indices):
    raise ValueError('indices should be a 1D vector with int32 or uint32 type.')
  if not is_int32_like(indptr):
    raise ValueError('indptr should be a 1D vector with int32 or uint32 type.')
  if events.ndim != 1:
    raise ValueError('events should be a 1D vector.')
  if len(shape) != 2:
    raise ValueError('shape should be a length-2 tuple.')
  if transpose:
    if events.shape[0] != shape[0]:
      raise ValueError(f'Shape mismatch, vec ({events.shape[0]},) @ mat {shape}.')
  else:
    if events.shape[0] != shape[1]:
      raise ValueError(f'Shape mismatch, mat {shape} @ vec ({events.shape[0]},).')
  if indptr.shape[0] != shape[0] + 1:
    raise ValueError(f'shape {shape} does not match the given indptr {tuple(indptr.shape)}.')
  shape = (int(shape[0]), int(shape[1]))
  data, indices, indptr, events = map(contiguous, (data, indices, indptr, events))
  _target_name(data, events)  # dtype errors before autograd machinery
  if torch.is_grad_enabled() and (data.requires_grad or events.requires_grad):
    return _EventCSRMatvec.apply(data, indices, indptr, events, shape, bool(transpose))
  return event_csr_matvec_raw(data, indices, indptr, events, shape=shape, transpose=bool(transpose))


_NONZERO_SUFFIX = {torch.bool: '_bool', torch.int32: '_int', torch.int64: '_long', torch.float32: '_float',
                   torch.float64: '_double'}


def event_info(events: torch.Tensor):
  """Collect event information: the event indices and the event number
  (mirrors brainpylib/_src/event_ops/event_info_collection.py:24-45).

  Parameters
  ----------
  events: tensor
    A 1-D vector (bool, int32, int64, float32 or float64); its non-zero entries are the events.
    A 2-D ``(batch, size)`` array is processed row by row (what ``vmap`` gives in the reference).

  Returns
  -------
  res: tuple
    ``(event_ids, event_num)``: int32 indices of the events in ASCENDING order padded with -1
    (same shape as ``events``), and their count (shape ``()`` or ``(batch,)``).  The reference's
    GPU kernel returns the same set of indices in an arbitrary order.
  """
  events = as_tensor(events, device_of(events))
  if events.ndim not in (1, 2):
    raise TypeError('Only support 1D boolean vector.')
  if events.dtype not in _NONZERO_SUFFIX:
    raise ValueError(f'unsupported events dtype {events.dtype}')
  if events.device.type != 'cuda':
    raise GPUOperatorNotFound(f'nonzero (operands are on {events.device}, a CUDA device is required)')
  events = contiguous(events)
  batch, size = (1, events.shape[0]) if events.ndim == 1 else events.shape
  name = 'nonzero' + _NONZERO_SUFFIX[events.dtype]
  opaque = gpu_ops.build_nonzero_descriptor(size, batch)
  ids = torch.empty(events.shape, dtype=torch.int32, device=events.device)
  num = torch.empty(batch, dtype=torch.int32, device=events.device)
  ws = _workspace(events.device, _lib.workspace_bytes(name, opaque))
  _lib.call(name, [events, ids, num, ws], opaque, device=events.device)
  return ids, (num[0] if events.ndim == 1 else num)
