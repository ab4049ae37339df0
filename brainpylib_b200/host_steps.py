"""Runs of many steps over spike trains that live in HOST memory (no counterpart in the reference, whose callers
hand one device array per call to ``event_csr_matvec``, brainpylib/_src/event_ops/event_csr_matvec.py:30-102).

:class:`HostSteps` computes ``event_csr_matvec(data, indices, indptr, events[s], shape=shape, transpose=True)`` for
every step ``s`` of a pinned host array of spike vectors and leaves every result in a pinned host array: the copy
in, the launch and the copy out of neighbouring steps overlap on three streams, and the library enqueues the whole
run in one native call (``bpl_run_host_steps``).  The multi-GPU form is ``PushExchange.run_host_steps``."""
import ctypes

import torch

from . import _lib, event_ops, gpu_ops
from .errors import GPUOperatorNotFound


def _pinned(t, what):
  if not isinstance(t, torch.Tensor) or t.device.type != 'cpu' or not t.is_pinned() or not t.is_contiguous():
    raise ValueError(f'{what} must be a contiguous tensor in pinned host memory')


def _ring(tensors):
  return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


class HostSteps:
  """``matrix``: ``(data, indices, indptr)`` of a CSR matrix on the GPU, or a
  :class:`brainpylib_b200.event_ops.ColumnBlockedCSR` made from one; ``events_dtype``: bool or float32."""

  def __init__(self, matrix, *, shape, events_dtype=torch.float32, group=3):
    """``group``: steps between cross-stream synchronisation points (1..16); the device rings hold ``3 * group``
    spike, result and workspace buffers."""
    n_row, n_col = int(shape[0]), int(shape[1])
    if not 1 <= int(group) <= 16:
      raise ValueError('group must be in 1..16')
    self.group = int(group)
    if events_dtype not in (torch.bool, torch.float32):
      raise ValueError('events must be bool or float32')
    suffix = 'bool' if events_dtype == torch.bool else 'float'
    if isinstance(matrix, event_ops.ColumnBlockedCSR):
      if matrix.shape != (n_row, n_col):
        raise ValueError(f'the prepared matrix has shape {matrix.shape}, not {(n_row, n_col)}')
      fixed = [matrix.groups, matrix.offsets]
      self.name = f'event_cbcsr_matvec_heter_float_{suffix}'
      self.opaque = event_ops._cb_descriptor(n_row, n_col, matrix.block_width, matrix.scale_log2, matrix.team_lanes_log2)
    else:
      data, indices, indptr = matrix
      if data.dtype != torch.float32 or indices.dtype != torch.int32 or indptr.dtype != torch.int32:
        raise TypeError('float32 weights and int32 indices / indptr are required')
      if indptr.numel() != n_row + 1 or data.numel() not in (1, indices.numel()):
        raise ValueError('indptr must have n_row + 1 entries and data one weight, or one per stored index')
      fixed = [data, indices, indptr]
      self.name = f"event_csr_matvec_{'homo' if data.numel() == 1 else 'heter'}_float_{suffix}"
      self.opaque = gpu_ops.build_twouint_onebool_descriptor(n_row, n_col, True)
    device = fixed[0].device
    if device.type != 'cuda':
      raise GPUOperatorNotFound(f'{self.name} (operands are on {device}, a CUDA device is required)')
    for t in fixed:
      if t.device != device or not t.is_contiguous():
        raise ValueError('the matrix must be contiguous and on one device')
    self.device, self.shape, self.events_dtype, self._fixed = device, (n_row, n_col), events_dtype, fixed
    ring = 3 * self.group
    self._ev = [torch.empty(n_row, dtype=events_dtype, device=device) for _ in range(ring)]
    self._y = [torch.empty(n_col, dtype=torch.float32, device=device) for _ in range(ring)]
    ws_bytes = _lib.workspace_bytes(self.name, self.opaque)
    self._ws = [torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device) for _ in range(ring)]
    self._streams = [torch.cuda.Stream(device) for _ in range(3)]
    n = len(fixed)
    self._buffers = (ctypes.c_void_p * (n + 3))(*[t.data_ptr() for t in fixed], self._ev[0].data_ptr(),
                                                 self._y[0].data_ptr(), self._ws[0].data_ptr())
    self._n = n
    self._fn = _lib.lib().bpl_run_host_steps
    self._fn.restype = None
    self._fn.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                         ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32,
                         ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint32,
                         ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]

  def run(self, host_events: torch.Tensor, host_out: torch.Tensor) -> float:
    """``host_events``: ``(n_steps, n_row)`` pinned; ``host_out``: ``(slots, n_col)`` pinned float32, step ``s`` lands
    in row ``s % slots``.  Blocks until the run is complete; returns the milliseconds the device spent on it (CUDA
    events on the compute stream around the whole run)."""
    n_row, n_col = self.shape
    _pinned(host_events, 'host_events')
    _pinned(host_out, 'host_out')
    if host_events.dtype != self.events_dtype or host_events.ndim != 2 or host_events.shape[1] != n_row:
      raise ValueError(f'host_events must be (n_steps, {n_row}) of {self.events_dtype}')
    if host_out.dtype != torch.float32 or host_out.ndim != 2 or host_out.shape[1] != n_col or host_out.shape[0] < 1:
      raise ValueError(f'host_out must be (slots, {n_col}) float32')
    s_in, s_c, s_out = self._streams
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.device(self.device):
      s_c.wait_stream(torch.cuda.current_stream(self.device))
      e0.record(s_c)
      n = self._n
      self._fn(self.name.encode(), self.opaque, len(self.opaque), self._buffers, n + 3, n, n + 1, n + 2, _ring(self._ev),
               _ring(self._y), _ring(self._ws), self.group, host_events.data_ptr(), host_events.shape[1] * host_events.element_size(),
               host_out.data_ptr(), n_col * 4, host_out.shape[0], host_events.shape[0], s_in.cuda_stream, s_c.cuda_stream,
               s_out.cuda_stream)
      e1.record(s_c)
      _lib.check_status()
      s_c.synchronize()
    return e0.elapsed_time(e1)
