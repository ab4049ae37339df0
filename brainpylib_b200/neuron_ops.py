"""The caller's side of a simulation step, fused (no counterpart in brainpylib, whose operators stop at the
product): ``lif_exp_step`` decays the synaptic conductances, adds the propagated input, integrates leaky
integrate-and-fire neurons and compacts the new spikes into the spike list that
``event_csr_matvec_from_list`` scatters from.  It is the update pattern of the reference's network example
(brainpylib/_src/op_register/tests/ei_net.py:47-72) with BrainPy's ``LIF`` / exponential-synapse rules restated
(BrainPy itself is not part of the reference tree):

    g_c  = g_c * exp(-dt / tau_syn_c) + y_c                     per synaptic channel c; y_c is then cleared
    I    = ext_input + sum_c g_c * (E_c - V)
    V'   = V_inf + (V - V_inf) * exp(-dt / tau),  V_inf = V_rest + R * I;   V' = V while (t - t_last) <= tau_ref
    spike = V' >= V_th;   t_last = t and V = V_reset where spike, else V = V'

A step of a recurrent network is then two launches: ``lif_exp_step`` and one list-driven scatter per projection.
"""
import ctypes
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib, gpu_ops
from .errors import GPUOperatorNotFound

__all__ = ['LifExpParams', 'lif_exp_step', 'spike_list_bytes', 'event_csr_matvec_from_list']


@dataclass
class LifExpParams:
  """Constants of the fused step.  The two decay factors are rounded to float32 once, here, and used as such by the
  kernel (and by any implementation it is compared with)."""
  dt: float
  tau_syn: Sequence[float]          # one per synaptic channel (1..4)
  E_rev: Sequence[float]
  ext_input: float = 0.0
  V_rest: float = -60.0
  V_th: float = -50.0
  V_reset: float = -60.0
  R: float = 1.0
  tau: float = 20.0
  tau_ref: float = 5.0
  syn_decay: np.ndarray = field(init=False)
  lif_decay: np.float32 = field(init=False)

  def __post_init__(self):
    if not (1 <= len(self.tau_syn) <= 4) or len(self.tau_syn) != len(self.E_rev):
      raise ValueError('1..4 synaptic channels, one time constant and one reversal potential each')
    self.syn_decay = np.exp(-np.float64(self.dt) / np.asarray(self.tau_syn, dtype=np.float64)).astype(np.float32)
    self.lif_decay = np.float32(np.exp(-np.float64(self.dt) / np.float64(self.tau)))

  @property
  def n_channels(self):
    return len(self.tau_syn)


def spike_list_bytes(n: int) -> int:
  """Size of the spike list of ``n`` neurons (the workspace layout of the transposed event product)."""
  return _lib.workspace_bytes('event_csr_matvec_heter_float_float', gpu_ops.build_twouint_onebool_descriptor(n, 1, True))


def _descriptor(p: LifExpParams, n: int, t: float) -> bytes:
  lib = _lib.lib()
  fn = lib.bpl_build_lif_exp_descriptor
  fn.restype = ctypes.c_size_t
  F = ctypes.c_float
  fn.argtypes = [ctypes.c_uint32, ctypes.c_uint32, F, ctypes.POINTER(F), ctypes.POINTER(F), F, F, F, F, F, F, F,
                 ctypes.c_void_p, ctypes.c_size_t]
  k = p.n_channels
  decay = (F * k)(*[float(v) for v in p.syn_decay])
  e_rev = (F * k)(*[float(np.float32(v)) for v in p.E_rev])
  buf = ctypes.create_string_buffer(128)
  size = fn(n, k, float(np.float32(t)), decay, e_rev, float(np.float32(p.ext_input)), float(np.float32(p.V_rest)),
            float(np.float32(p.V_th)), float(np.float32(p.V_reset)), float(np.float32(p.R)), float(p.lif_decay),
            float(np.float32(p.tau_ref)), buf, 128)
  if size == 0:
    raise ValueError('bad fused-step parameters')
  return buf.raw[:size]


def lif_exp_step(y: torch.Tensor, g: torch.Tensor, V: torch.Tensor, t_last: torch.Tensor, params: LifExpParams, t: float,
                 *, spikes: Optional[torch.Tensor] = None, spike_list: Optional[torch.Tensor] = None):
  """One fused update of ``n`` neurons, in place.

  ``y``, ``g``: float32 ``(K, n)`` (or ``(n,)`` for one channel): propagated input (consumed, then ZERO-FILLED so
  that the next list-driven product can accumulate into it) and conductances.  ``V``, ``t_last``: float32 ``(n,)``.
  Returns ``(spikes, spike_list)``: float32 0/1 ``(n,)`` and the uint8 buffer holding the compacted spike list
  (``spike_list_bytes(n)`` bytes) for :func:`event_csr_matvec_from_list`; both are allocated when not given."""
  n = V.shape[0]
  k = params.n_channels
  if V.device.type != 'cuda':
    raise GPUOperatorNotFound(f'lif_exp_step_float (operands are on {V.device}, a CUDA device is required)')
  for name, a, shape in (('y', y, (k, n)), ('g', g, (k, n)), ('V', V, (n,)), ('t_last', t_last, (n,))):
    ok_shape = tuple(a.shape) == shape or (k == 1 and tuple(a.shape) == (n,))
    if a.dtype != torch.float32 or not ok_shape or not a.is_contiguous() or a.device != V.device:
      raise ValueError(f'{name} must be a contiguous float32 tensor of shape {shape} on the device of V')
  if spikes is None:
    spikes = torch.empty(n, dtype=torch.float32, device=V.device)
  if spike_list is None:
    spike_list = torch.empty(spike_list_bytes(n), dtype=torch.uint8, device=V.device)
  elif spike_list.numel() * spike_list.element_size() < spike_list_bytes(n):
    raise ValueError('spike_list is too small')
  _lib.call('lif_exp_step_float', [y, g, V, t_last, spikes, spike_list], _descriptor(params, n, t), device=V.device)
  return spikes, spike_list


def event_csr_matvec_from_list(data, indices, indptr, spike_list, y, *, shape, prepared=None):
  """``y += A^T spikes`` from the compacted spike list of :func:`lif_exp_step` (``y`` float32 ``(shape[1],)``, already
  zero: ``lif_exp_step`` leaves it so).  With ``prepared`` (see ``prepare_event_csr``) the product runs on the
  column-blocked layout and the CSR operands may be ``None``."""
  from .event_ops import _cb_descriptor, ColumnBlockedCSR
  n_row, n_col = int(shape[0]), int(shape[1])
  if y.dtype != torch.float32 or y.numel() != n_col or not y.is_contiguous():
    raise ValueError('y must be a contiguous float32 vector of shape[1] entries')
  if spike_list.numel() * spike_list.element_size() < spike_list_bytes(n_row):
    raise ValueError('spike_list is too small for shape[0] rows')
  if prepared is not None:
    if not isinstance(prepared, ColumnBlockedCSR) or prepared.shape != (n_row, n_col):
      raise ValueError('prepared does not describe a matrix of this shape')
    opaque = _cb_descriptor(n_row, n_col, prepared.block_width, prepared.scale_log2, prepared.team_lanes_log2)
    _lib.call('event_cbcsr_matvec_list_heter_float', [prepared.groups, prepared.offsets, spike_list, y], opaque,
              device=y.device)
    return y
  if data.dtype != torch.float32 or data.numel() != indices.numel() or indptr.numel() != n_row + 1:
    raise ValueError('the list-driven CSR product takes heterogeneous float32 weights and shape[0] + 1 row pointers')
  if n_row > 1024 * 4096:
    raise ValueError('more than 4,194,304 rows')
  n_chunks = -(-n_row // 4096)
  opaque = gpu_ops.build_triple_size_descriptor(n_row, n_col, n_chunks)
  _lib.call('event_csr_matvec_list_heter_float', [data, indices, indptr, spike_list, y], opaque, device=y.device)
  return y
