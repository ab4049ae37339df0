"""The entry point for callers that cannot allocate: `event_csr_matvec_heter_float_float_noalloc`.

An XLA custom call (or any code running while a stream is being captured) gets only the buffers
its framework planned and must not call cudaMalloc; this entry point therefore takes the
reference's plain five-buffer list and keeps its scratch in a fixed device array inside the
library.  The test drives it through the C ABI exactly as such a caller would (raw device
pointers, packed descriptor, a stream) and compares it with the regular entry point, which
receives its scratch as a workspace buffer.  Two calls in a row with different spikes check
that what the first call left in the shared scratch does not leak into the second.

Collected last on purpose (file name), so a run that stops at the first failure has already
run everything else.  Tolerance: the one used for every heterogeneous scatter here
(rtol 1e-5, atol 1e-5 * largest in-degree; the float atomics may add in any order).
"""
import ctypes

import numpy as np
import pytest
import torch

import cases
from brainpylib_b200 import _lib, gpu_ops
from oracle import cpu

pytestmark = pytest.mark.gpu


def call_raw(name, buffers, opaque, stream):
  fn = getattr(_lib.lib(), name)
  fn.restype = None
  fn.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p, ctypes.c_size_t]
  ptrs = (ctypes.c_void_p * len(buffers))(*[b.data_ptr() for b in buffers])
  fn(stream, ptrs, opaque, len(opaque))
  return _lib.lib().bpl_last_status(None, 0)


def test_noalloc_entry_matches_workspace_entry_twice(cuda):
  shape = (6000, 5000)
  data, indices, indptr, rng = cases.csr_case(shape, 0.02, 91)
  d_data, d_idx, d_ptr = (torch.as_tensor(a).to(cuda) for a in (data, indices, indptr))
  opaque = gpu_ops.build_twouint_onebool_descriptor(shape[0], shape[1], True)
  ws = torch.empty(_lib.workspace_bytes('event_csr_matvec_heter_float_float', opaque), dtype=torch.uint8, device=cuda)
  atol = 1e-5 * max(1, int(np.bincount(indices, minlength=shape[1]).max()))
  stream = torch.cuda.current_stream(cuda).cuda_stream
  _lib.lib().bpl_clear_status()
  for rate in (0.3, 0.02):      # the second call has fewer spikes: stale list entries must not be used
    events = torch.as_tensor((rng.random(shape[0]) < rate).astype(np.float32)).to(cuda)
    y_ws = torch.full((shape[1],), float('nan'), device=cuda)
    y_na = torch.full((shape[1],), float('nan'), device=cuda)
    assert call_raw('event_csr_matvec_heter_float_float', [d_data, d_idx, d_ptr, events, y_ws, ws], opaque, stream) == 0
    assert call_raw('event_csr_matvec_heter_float_float_noalloc', [d_data, d_idx, d_ptr, events, y_na], opaque,
                    stream) == 0
    torch.cuda.synchronize()
    assert torch.isfinite(y_na).all()
    torch.testing.assert_close(y_na, y_ws, rtol=1e-5, atol=atol)
    assert y_ws.abs().sum().item() > 0
    want = cpu.event_csr_matvec(data, indices, indptr, events.cpu().numpy(), shape=shape, transpose=True)
    np.testing.assert_allclose(y_na.cpu().numpy(), want, rtol=1e-5, atol=atol)     # and against the CPU oracle


def test_noalloc_entry_at_its_row_limit_unaligned_and_empty(cuda):
  """Exactly 2^21 rows (the whole fixed scratch), index / weight arrays that start 4 bytes off a 16-byte
  boundary (the element-wise kernel), and a matrix without rows: each against the CPU oracle."""
  lib = _lib.lib()
  stream = torch.cuda.current_stream(cuda).cuda_stream
  lib.bpl_clear_status()
  rng = np.random.default_rng(93)
  n_row, n_col = 1 << 21, 3000
  lens = np.zeros(n_row, dtype=np.int64)
  busy = rng.choice(n_row, 4000, replace=False)
  lens[busy] = rng.integers(1, 40, busy.shape[0])
  lens[-1] = 17                                   # the last row the scratch can list
  data, indices, indptr, rng = cases.ragged_csr(lens, n_col, 94)
  ev = np.zeros(n_row, dtype=np.float32)
  ev[busy[::2]] = 1.0
  ev[-1] = 3.0
  want = cpu.event_csr_matvec(data, indices, indptr, ev, shape=(n_row, n_col), transpose=True)
  atol = 1e-5 * max(1, int(np.bincount(indices, minlength=n_col).max()))
  # 16-byte aligned and shifted by one element
  for shift in (0, 1):
    d_data = torch.zeros(data.shape[0] + 4, device=cuda)[shift:shift + data.shape[0]].copy_(torch.as_tensor(data))
    d_idx = torch.zeros(indices.shape[0] + 4, dtype=torch.int32, device=cuda)[shift:shift + indices.shape[0]].copy_(
      torch.as_tensor(indices))
    assert (d_data.data_ptr() % 16 == 0) == (shift == 0)
    d_ptr, d_ev = torch.as_tensor(indptr).to(cuda), torch.as_tensor(ev).to(cuda)
    y = torch.full((n_col,), float('nan'), device=cuda)
    opaque = gpu_ops.build_twouint_onebool_descriptor(n_row, n_col, True)
    assert call_raw('event_csr_matvec_heter_float_float_noalloc', [d_data, d_idx, d_ptr, d_ev, y], opaque, stream) == 0
    torch.cuda.synchronize()
    np.testing.assert_allclose(y.cpu().numpy(), want, rtol=1e-5, atol=atol)
  # no rows: the output is zero-filled and nothing else runs
  y = torch.full((5,), float('nan'), device=cuda)
  empty = torch.zeros(1, dtype=torch.int32, device=cuda)
  opaque = gpu_ops.build_twouint_onebool_descriptor(0, 5, True)
  assert call_raw('event_csr_matvec_heter_float_float_noalloc', [y, empty, empty, y, y], opaque, stream) == 0
  torch.cuda.synchronize()
  assert torch.equal(y, torch.zeros_like(y))


def test_noalloc_entry_rejects_what_it_cannot_do(cuda):
  lib = _lib.lib()
  lib.bpl_noalloc_max_rows.restype = ctypes.c_uint32
  limit = lib.bpl_noalloc_max_rows()
  assert limit == 1 << 21
  dummy = torch.zeros(8, device=cuda)
  lib.bpl_clear_status()
  too_big = gpu_ops.build_twouint_onebool_descriptor(limit + 1, 10, True)
  assert call_raw('event_csr_matvec_heter_float_float_noalloc', [dummy] * 5, too_big, None) == 4   # BPL_ERR_TOO_LARGE
  msg = ctypes.create_string_buffer(256)
  lib.bpl_last_status(msg, 256)
  assert b'2097152' in msg.value
  lib.bpl_clear_status()
  not_transposed = gpu_ops.build_twouint_onebool_descriptor(10, 10, False)
  assert call_raw('event_csr_matvec_heter_float_float_noalloc', [dummy] * 5, not_transposed, None) == 3
  lib.bpl_clear_status()
  assert call_raw('event_csr_matvec_heter_float_float_noalloc', [dummy] * 5, b'abc', None) == 1
  lib.bpl_clear_status()
  torch.cuda.synchronize()
