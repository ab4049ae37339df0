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

__all__ = ['event_csr_matvec', 'event_info', 'ColumnBlockedCSR', 'csr_to_column_blocked', 'event_cbcsr_matvec']

_workspaces = {}
_retired_workspaces = []


def _workspace(device, nbytes):
  """A per-(device, stream) scratch tensor, grown on demand.  Kernels of one stream run
  in order, so one buffer per stream is safe to reuse.  A buffer that is outgrown is kept
  alive: a captured CUDA graph may still hold its address."""
  key = (device.index, torch.cuda.current_stream(device).cuda_stream)
  ws = _workspaces.get(key)
  if ws is None or ws.numel() < nbytes:
    if ws is not None:
      _retired_workspaces.append(ws)
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


# --------------------------------------------------------------------------------------------------
# Column-blocked CSR: a second storage format for the transposed event product
# --------------------------------------------------------------------------------------------------
# No counterpart in the reference.  The plain CSR scatter is bound by scattered reductions in L2
# (one 32-byte sector operation per synapse).  Cutting the post-synaptic neurons into blocks narrow
# enough for one block of the output to live in a CTA's shared memory moves the accumulation out of
# L2.  The format stays row-major: every CSR row keeps its place and its length, but its entries are
# grouped by column block (stable, so the CSR order survives inside a group), column ids become
# 16-bit offsets into their block, and a per-row table says where each block's group starts.  The
# conversion is done once per matrix; the operator that consumes the format is stateless.

class ColumnBlockedCSR:
  """``offsets`` int32 ``(n_row, n_blocks + 1)``: ``offsets[r, b] .. offsets[r, b + 1]`` are row ``r``'s
               synapses that target block ``b`` (absolute positions; ``offsets[r, 0] == indptr[r]``,
               ``offsets[r, n_blocks] == indptr[r + 1]``),
  ``cols``    int16 storage of uint16 local column ids (column = ``b * block_width + cols``),
  ``data``    weights in the same order, ``shape`` the matrix shape, ``block_width`` columns per block."""

  def __init__(self, offsets, cols, data, shape, block_width):
    self.offsets, self.cols, self.data = offsets, cols, data
    self.shape = (int(shape[0]), int(shape[1]))
    self.block_width = int(block_width)
    self.n_blocks = int(offsets.shape[1]) - 1

  def nbytes(self):
    return sum(t.numel() * t.element_size() for t in (self.offsets, self.cols, self.data))


def default_block_width(n_col, device=None):
  """Columns per block: as many blocks as give every SM one CTA when each block is shared by 4 CTAs,
  capped by what fits a CTA's shared memory next to the row-pointer cache (45056 floats = 176 KB)."""
  sms = torch.cuda.get_device_properties(device).multi_processor_count if torch.cuda.is_available() else 148
  n_blocks = max(1, sms // 4)
  width = -(-n_col // n_blocks)
  width = min(max(width, 1024), 45056)
  return -(-width // 32) * 32


def csr_to_column_blocked(data, indices, indptr, *, shape, block_width=None, rows_per_pass=100_000):
  """Re-lay a CSR matrix (heterogeneous float32 weights, int32 ids) into :class:`ColumnBlockedCSR`.

  Runs on the device of the operands in passes of ``rows_per_pass`` rows (one stable sort per pass).
  Needs the matrix to have fewer than 2^31 entries."""
  n_row, n_col = int(shape[0]), int(shape[1])
  device = indices.device
  if block_width is None:
    block_width = default_block_width(n_col, device)
  if not (0 < block_width <= 65536):
    raise ValueError('block_width must be in 1..65536 (local column ids are 16 bits)')
  nse = int(indices.shape[0])
  if nse >= 2 ** 31:
    raise ValueError('more than 2^31 - 1 stored entries')
  n_blocks = max(1, -(-n_col // block_width))
  indptr64 = indptr.to(torch.int64)
  lengths = indptr64[1:] - indptr64[:-1]
  offsets = torch.empty((n_row, n_blocks + 1), dtype=torch.int32, device=device)
  cols = torch.empty(nse, dtype=torch.int16, device=device)
  vals = torch.empty(nse, dtype=data.dtype, device=device)
  for r0 in range(0, n_row, rows_per_pass):
    r1 = min(n_row, r0 + rows_per_pass)
    a, b = int(indptr64[r0]), int(indptr64[r1])
    idx = indices[a:b].to(torch.int64)
    blk = idx // block_width
    row = torch.repeat_interleave(torch.arange(r1 - r0, device=device), lengths[r0:r1])
    key = row * n_blocks + blk
    counts = torch.bincount(key, minlength=(r1 - r0) * n_blocks).view(r1 - r0, n_blocks)
    ends = torch.cumsum(counts.view(-1), 0).view(r1 - r0, n_blocks) + a
    offsets[r0:r1, 1:] = ends.to(torch.int32)
    offsets[r0:r1, 0] = indptr64[r0:r1].to(torch.int32)
    if b > a:
      order = torch.sort(key, stable=True).indices
      # uint16 stored in int16: values >= 32768 wrap, the kernel reads them back as unsigned
      cols[a:b] = (idx - blk * block_width)[order].to(torch.int32).to(torch.int16)
      vals[a:b] = data[a:b][order]
      del order
    del idx, blk, row, key, counts, ends
  return ColumnBlockedCSR(offsets, cols, vals, shape, block_width)


def event_cbcsr_matvec_raw(blocked: ColumnBlockedCSR, events, *, out=None, workspace=None):
  """``y = A^T events`` on a :class:`ColumnBlockedCSR` (heterogeneous float32 weights; bool or float32
  events).  Target ``event_cbcsr_matvec_heter_float_{bool,float}``."""
  n_row, n_col = blocked.shape
  if events.dtype == torch.bool:
    name = 'event_cbcsr_matvec_heter_float_bool'
  elif events.dtype == torch.float32:
    name = 'event_cbcsr_matvec_heter_float_float'
  else:
    raise ValueError('events must be bool or float32')
  if blocked.data.dtype != torch.float32:
    raise TypeError('column-blocked CSR holds float32 weights')
  if events.device.type != 'cuda':
    raise GPUOperatorNotFound(f'{name} (operands are on {events.device}, a CUDA device is required)')
  opaque = _cb_descriptor(n_row, n_col, blocked.block_width)
  if out is None:
    out = torch.empty(n_col, dtype=torch.float32, device=events.device)
  if workspace is None:
    workspace = _workspace(events.device, _lib.workspace_bytes(name, opaque))
  _lib.call(name, [blocked.data, blocked.cols, blocked.offsets, events, out, workspace], opaque, device=events.device)
  return out


def _cb_descriptor(n_row, n_col, block_width):
  return gpu_ops.build_triple_size_descriptor(n_row, n_col, block_width)


def event_cbcsr_matvec(blocked: ColumnBlockedCSR, events: torch.Tensor) -> torch.Tensor:
  """Transposed event product ``y[c] = sum of w over the synapses (r, c) with events[r] != 0`` on a
  matrix converted once with :func:`csr_to_column_blocked`.  Same result as
  ``event_csr_matvec(data, indices, indptr, events, shape=shape, transpose=True)`` up to the order
  of the floating-point additions."""
  events = as_tensor(events, blocked.data.device)
  if events.ndim != 1 or events.shape[0] != blocked.shape[0]:
    raise ValueError(f'Shape mismatch, vec ({tuple(events.shape)},) @ mat {blocked.shape}.')
  return event_cbcsr_matvec_raw(blocked, contiguous(events))
