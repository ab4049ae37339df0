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
from ._checks import as_tensor, contiguous, device_of, float_suffix, is_int32_like, loop_vmap

__all__ = ['event_csr_matvec', 'event_info', 'ColumnBlockedCSR', 'csr_to_column_blocked', 'prepare_event_csr',
           'event_cbcsr_matvec']

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
  """Differentiation and batching rules of brainpylib/_src/event_ops/event_csr_matvec.py:439-463.

  Reverse mode (the transpose rules, :447-463), written as the vector-Jacobian product torch asks for:
  * w.r.t. ``events``: ``A^T ct`` (or ``A ct``), i.e. the dense CSR product with the opposite ``transpose``;
  * w.r.t. homogeneous ``data``: ``<ct, op(1, events)>``;
  * w.r.t. heterogeneous ``data``: ``events[row] * ct[col]`` if transpose else ``events[col] * ct[row]``.
  Forward mode (the JVP rules, :439-444): data tangent -> the same event product on ``data_dot``; events tangent
  -> the dense CSR product of ``data`` with ``events_dot``, same ``transpose``.
  Batching: a loop over the batch (what `register_general_batching` does in the reference)."""

  @staticmethod
  def forward(data, indices, indptr, events, shape, transpose):
    return event_csr_matvec_raw(data, indices, indptr, events, shape=shape, transpose=transpose)

  @staticmethod
  def setup_context(ctx, inputs, output):
    data, indices, indptr, events, shape, transpose = inputs
    ctx.save_for_backward(data, indices, indptr, events)
    ctx.save_for_forward(data, indices, indptr, events)
    ctx.shape, ctx.transpose = shape, transpose

  # The rules call the operators through their autograd functions, not the raw kernels: under torch.func
  # transforms the tangents and cotangents arrive wrapped, and only `apply` knows how to unwrap them.
  @staticmethod
  def backward(ctx, ct):
    from .sparse_ops import _CSRMatvec, csr_to_coo
    data, indices, indptr, events = ctx.saved_tensors
    shape, transpose = ctx.shape, ctx.transpose
    ct = contiguous(ct)
    g_data = g_events = None
    if ctx.needs_input_grad[0]:
      if data.shape[0] == 1:
        ones = torch.ones(1, dtype=data.dtype, device=data.device)
        r = _EventCSRMatvec.apply(ones, indices, indptr, events, shape, transpose)
        g_data = torch.dot(ct, r).reshape(1)
      else:
        row, col = csr_to_coo(indices, indptr)
        ev = events.to(data.dtype)
        g_data = ev[row] * ct[col] if transpose else ev[col] * ct[row]
    if ctx.needs_input_grad[3]:
      g_events = _CSRMatvec.apply(data, indices, indptr, ct, shape, not transpose, 'vector')
    return g_data, None, None, g_events, None, None

  @staticmethod
  def jvp(ctx, data_dot, _indices, _indptr, events_dot, _shape, _transpose):
    from .sparse_ops import _CSRMatvec
    data, indices, indptr, events = ctx.saved_tensors
    shape, transpose = ctx.shape, ctx.transpose
    tangent = None
    if data_dot is not None:
      tangent = _EventCSRMatvec.apply(contiguous(data_dot), indices, indptr, events, shape, transpose)
    if events_dot is not None:
      t = _CSRMatvec.apply(data, indices, indptr, contiguous(events_dot.to(data.dtype)), shape, transpose, 'vector')
      tangent = t if tangent is None else tangent + t
    return tangent

  @staticmethod
  def vmap(info, in_dims, data, indices, indptr, events, shape, transpose):
    return loop_vmap(_EventCSRMatvec.apply, info, in_dims, (data, indices, indptr, events, shape, transpose))


def event_csr_matvec(
    data: Union[float, torch.Tensor],
    indices: torch.Tensor,
    indptr: torch.Tensor,
    events: torch.Tensor,
    *,
    shape: Tuple[int, int],
    transpose: bool = False,
    prepared=None
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
  prepared: ColumnBlockedCSR, optional
    Not in the reference.  The same matrix converted once with :func:`prepare_event_csr`; with
    ``transpose=True``, float32 weights and no gradient requested the product then runs on that layout
    (accumulation in shared memory instead of scattered reductions in L2).  The CSR operands are still
    checked and are what differentiation uses.  The sums of one output are grouped differently, so the
    result agrees with the plain path to rounding, not bit for bit.

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
  if prepared is not None and transpose and data.dtype == torch.float32 and \
      not (torch.is_grad_enabled() and (data.requires_grad or events.requires_grad)):
    if not isinstance(prepared, ColumnBlockedCSR) or prepared.shape != shape or prepared.nse != indices.shape[0]:
      raise ValueError('prepared does not describe this matrix (built from another shape or entry count).')
    return event_cbcsr_matvec_raw(prepared, events)
  # always through the autograd function: it carries the reverse-mode, forward-mode and batching rules
  return _EventCSRMatvec.apply(data, indices, indptr, events, shape, bool(transpose))


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
# Column-blocked matrix: a prepared storage format for the transposed event product
# --------------------------------------------------------------------------------------------------
# No counterpart in the reference.  The plain CSR scatter is bound by scattered reductions in L2
# (one 32-byte sector operation per synapse).  Cutting the post-synaptic neurons into blocks narrow
# enough for one block of the output to live in a CTA's shared memory moves the accumulation out of
# L2.  The format stays row-major: the synapses of a row lie together, grouped by column block (the
# CSR order survives inside a group), in records of 8 synapses (8 float32 weights, then 8 16-bit
# column offsets into the block; a segment is padded with zero-weight synapses to whole records), and
# a per-row table says where each block's segment starts.  The conversion runs once per matrix, on the
# GPU (csrc/cbcsr_build.cu); the operator that consumes the format is stateless.

CB_GROUP_BYTES = 48
CB_MAX_WIDTH = 32256


class ColumnBlockedCSR:
  """``groups``  uint8 ``(48 * n_groups,)``: records of 8 synapses, ``float32 w[8]`` then ``uint16 c[8]``
               (column = ``col_range[0] + b * block_width + c``),
  ``offsets`` int32 storage of uint32 ``(n_row, n_blocks + 1)``: records ``offsets[r, b] .. offsets[r, b + 1]``
               hold row ``r``'s synapses that target block ``b``,
  ``shape``   the shape of the matrix this object multiplies by (``n_row``, columns kept),
  ``col_range`` the columns ``[lo, hi)`` of the source matrix that were kept (a rank's shard), re-based to ``lo``."""

  def __init__(self, groups, offsets, shape, block_width, col_range=None, nse=None, scale_log2=None):
    self.groups, self.offsets = groups, offsets
    # lanes (= records per round) one (row, block) segment gets in the kernel: the smallest of 4, 8, 16, 32 that
    # covers an average segment with some room (longer segments take more rounds)
    segments = max(1, int(offsets.shape[0]) * max(1, int(offsets.shape[1]) - 1))
    mean_groups = (groups.numel() // CB_GROUP_BYTES) / segments
    self.team_lanes_log2 = 2 if mean_groups <= 3.6 else 3 if mean_groups <= 7.0 else 4 if mean_groups <= 14.0 else 5
    self.scale_log2 = scale_log2     # None: float accumulators; k: 32-bit fixed point, 2^k units per 1.0
    self.shape = (int(shape[0]), int(shape[1]))
    self.block_width = int(block_width)
    self.n_blocks = int(offsets.shape[1]) - 1
    self.col_range = (0, self.shape[1]) if col_range is None else (int(col_range[0]), int(col_range[1]))
    self.nse = nse

  @property
  def n_groups(self):
    return self.groups.numel() // CB_GROUP_BYTES

  def nbytes(self):
    return sum(t.numel() * t.element_size() for t in (self.groups, self.offsets))


def default_block_width(n_col, device=None, reserve=0):
  """Columns per block.  The kernel gives every column block ``P = floor(SMs / n_blocks)`` CTAs, one per SM, so the
  choice is the number of blocks: at least ``n_col / 20480`` (a block's slice of the output and the copy buffers
  per warp must fit a CTA's shared memory; wide blocks mean long row segments, which stream best), and more only
  where that fills at least 10 % more of the SMs.  ``reserve``: SMs to leave free (the one-launch sharded step runs
  up to four exchanging blocks beside the scatter).  At least 1024 columns, a multiple of 32."""
  sms = torch.cuda.get_device_properties(device).multi_processor_count if torch.cuda.is_available() else 148
  sms = max(1, sms - reserve)
  least = max(1, -(-n_col // 20480))
  best, best_ctas = least, least * max(1, sms // least)
  for n_blocks in range(least + 1, min(2 * least, sms) + 1):
    ctas = n_blocks * (sms // n_blocks)
    if ctas * 100 >= best_ctas * 110:
      best, best_ctas = n_blocks, ctas
  width = max(-(-n_col // best), 1024)
  return min(-(-width // 32) * 32, 20480)


def check_block_width(block_width):
  if not (32 <= block_width <= CB_MAX_WIDTH) or block_width % 32 != 0:
    raise ValueError(f'block_width must be a multiple of 32 in 32..{CB_MAX_WIDTH}, got {block_width}')


def csr_to_column_blocked(data, indices, indptr, *, shape, block_width=None, col_range=None, accumulate='float'):
  """Re-lay a CSR matrix (float32 weights, heterogeneous or one shared value; int32 ids) into
  :class:`ColumnBlockedCSR` on the GPU that holds it.

  ``col_range = (lo, hi)`` keeps only the synapses whose target lies in ``[lo, hi)`` and re-bases them
  to ``lo``: one rank's shard of a matrix partitioned by post-synaptic neuron.  Two kernel passes over
  the matrix and one host read of the result size; needs fewer than 2^32 records of 8 synapses.

  ``accumulate='float'`` (default): the kernel sums in float32, like the plain operator.
  ``accumulate='fixed'``: it sums in 32-bit fixed point, which the hardware adds in shared memory several
  times faster than floats.  One more pass finds ``M``, the largest sum of ``|w|`` over any column, and the
  unit is ``2^-k`` with ``k = floor(log2(2^30 / M))``: no spike pattern can overflow.  Every weight is
  rounded to a multiple of the unit, so an output fed by ``n`` active synapses is off by at most
  ``n * 2^-(k+1)``, about ``n * M * 2^-31``; the integer sum inside a CTA is exact and order-independent, and
  the only float32 roundings left are the conversion of each CTA's sum and the addition of the few CTAs that
  share a column block (so two launches that split the rows differently may differ in the last bit).  With
  weights of similar magnitude that is the accuracy of float32 summation; a column that mixes huge and tiny
  weights keeps the tiny ones only to that absolute step."""
  import ctypes
  n_row, n_col = int(shape[0]), int(shape[1])
  lo, hi = (0, n_col) if col_range is None else (int(col_range[0]), int(col_range[1]))
  if not (0 <= lo <= hi <= n_col):
    raise ValueError(f'col_range {col_range} does not lie inside 0..{n_col}')
  device = indices.device
  if device.type != 'cuda':
    raise GPUOperatorNotFound(f'column-blocked build (operands are on {device}, a CUDA device is required)')
  if block_width is None:
    block_width = default_block_width(hi - lo, device)
  block_width = int(block_width)
  check_block_width(block_width)
  if data.dtype != torch.float32:
    raise TypeError('the column-blocked format holds float32 weights')
  if not (is_int32_like(indices) and is_int32_like(indptr)):
    raise ValueError('indices and indptr should be int32 or uint32 vectors.')
  if indptr.shape[0] != n_row + 1:
    raise ValueError(f'shape {shape} does not match the given indptr {tuple(indptr.shape)}.')
  if data.shape[0] not in (1, indices.shape[0]):
    raise ValueError('The size of data should be 1 or be consistent with indices.')
  data, indices, indptr = map(contiguous, (data, indices, indptr))
  lib = _lib.lib()
  lib.bpl_cbcsr_build_workspace_bytes.restype = ctypes.c_size_t
  lib.bpl_cbcsr_build_workspace_bytes.argtypes = [ctypes.c_uint32]
  lib.bpl_cbcsr_n_blocks.restype = ctypes.c_uint32
  lib.bpl_cbcsr_n_blocks.argtypes = [ctypes.c_uint32, ctypes.c_uint32]
  lib.bpl_cbcsr_plan.restype = None
  lib.bpl_cbcsr_plan.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32,
                                 ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p]
  lib.bpl_cbcsr_fill.restype = None
  lib.bpl_cbcsr_fill.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                 ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p,
                                 ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_int]
  n_blocks = int(lib.bpl_cbcsr_n_blocks(hi - lo, block_width))
  if n_blocks > 1024:
    raise ValueError(f'{n_blocks} column blocks; at most 1024 (use a wider block)')
  with torch.cuda.device(device):
    stream = torch.cuda.current_stream(device).cuda_stream
    offsets = torch.empty((n_row, n_blocks + 1), dtype=torch.int32, device=device)
    ws = torch.empty(int(lib.bpl_cbcsr_build_workspace_bytes(n_row)) // 8 + 1, dtype=torch.int64, device=device)
    lib.bpl_cbcsr_plan(stream, indices.data_ptr(), indptr.data_ptr(), n_row, lo, hi, block_width, offsets.data_ptr(),
                       ws.data_ptr())
    _lib.check_status()
    n_groups = int(ws[0].item())    # the one synchronisation of the build
    if n_groups >= 2 ** 32:
      raise ValueError('2^32 or more records of 8 synapses')
    homo = int(data.shape[0] == 1 and indices.shape[0] != 1)
    scale_log2 = None
    if accumulate == 'fixed':
      lib.bpl_cbcsr_max_column_abs_sum.restype = None
      lib.bpl_cbcsr_max_column_abs_sum.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                                   ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p,
                                                   ctypes.c_void_p]
      colsum = torch.empty(max(hi - lo, 1), dtype=torch.float32, device=device)
      biggest = torch.empty(1, dtype=torch.float32, device=device)
      lib.bpl_cbcsr_max_column_abs_sum(stream, data.data_ptr(), homo, indices.data_ptr(), int(indices.shape[0]), lo, hi,
                                       colsum.data_ptr(), biggest.data_ptr())
      _lib.check_status()
      scale_log2 = fixed_point_scale_log2(float(biggest.item()))
      del colsum
    elif accumulate != 'float':
      raise ValueError("accumulate must be 'float' or 'fixed'")
    groups = torch.empty(n_groups * CB_GROUP_BYTES, dtype=torch.uint8, device=device)
    lib.bpl_cbcsr_fill(stream, data.data_ptr(), homo, indices.data_ptr(), indptr.data_ptr(), n_row, lo, hi, block_width,
                       offsets.data_ptr(), ws.data_ptr(), groups.data_ptr(), n_groups,
                       0 if scale_log2 is None else 1, 0 if scale_log2 is None else scale_log2)
    _lib.check_status()
  return ColumnBlockedCSR(groups, offsets, (n_row, hi - lo), block_width, (lo, hi), nse=int(indices.shape[0]),
                          scale_log2=scale_log2)


def fixed_point_scale_log2(max_column_abs_sum: float) -> int:
  """``k`` such that a column whose ``|w|`` sum to ``max_column_abs_sum`` stays below 2^30 units of ``2^-k``."""
  import math
  if not math.isfinite(max_column_abs_sum):
    raise ValueError('the weights are not finite: fixed-point accumulation is not possible')
  if max_column_abs_sum <= 0.0:
    return 0
  return max(-100, min(100, math.floor(math.log2(2.0 ** 30 / max_column_abs_sum))))


prepare_event_csr = csr_to_column_blocked


def event_cbcsr_matvec_raw(blocked: ColumnBlockedCSR, events, *, out=None, workspace=None):
  """``y = A^T events`` on a :class:`ColumnBlockedCSR` (float32 weights; bool or float32 events).
  Target ``event_cbcsr_matvec_heter_float_{bool,float}``."""
  n_row, n_col = blocked.shape
  if events.dtype == torch.bool:
    name = 'event_cbcsr_matvec_heter_float_bool'
  elif events.dtype == torch.float32:
    name = 'event_cbcsr_matvec_heter_float_float'
  else:
    raise ValueError('events must be bool or float32')
  if events.device.type != 'cuda':
    raise GPUOperatorNotFound(f'{name} (operands are on {events.device}, a CUDA device is required)')
  opaque = _cb_descriptor(n_row, n_col, blocked.block_width, blocked.scale_log2, blocked.team_lanes_log2)
  if out is None:
    out = torch.empty(n_col, dtype=torch.float32, device=events.device)
  if workspace is None:
    workspace = _workspace(events.device, _lib.workspace_bytes(name, opaque))
  _lib.call(name, [blocked.groups, blocked.offsets, events, out, workspace], opaque, device=events.device)
  return out


def _cb_descriptor(n_row, n_col, block_width, scale_log2=None, team_lanes_log2=2):
  import struct
  return struct.pack('<IIIiiI', n_row, n_col, block_width, 0 if scale_log2 is None else 1,
                     0 if scale_log2 is None else int(scale_log2), int(team_lanes_log2))


def event_cbcsr_matvec(blocked: ColumnBlockedCSR, events: torch.Tensor) -> torch.Tensor:
  """Transposed event product ``y[c] = sum of w over the synapses (r, c) with events[r] != 0`` on a
  matrix converted once with :func:`csr_to_column_blocked`.  Same result as
  ``event_csr_matvec(data, indices, indptr, events, shape=shape, transpose=True)`` up to the order
  of the floating-point additions."""
  events = as_tensor(events, blocked.groups.device)
  if events.ndim != 1 or events.shape[0] != blocked.shape[0]:
    raise ValueError(f'Shape mismatch, vec ({tuple(events.shape)},) @ mat {blocked.shape}.')
  return event_cbcsr_matvec_raw(blocked, contiguous(events))
