"""ctypes binding of ``libbrainpylib_b200.so`` and the one call path every operator uses.

The library's entry points are XLA legacy custom-call targets
``void f(cudaStream_t, void** buffers, const char* opaque, size_t opaque_len)``;
torch only supplies device memory and the current stream.
"""
import ctypes
import functools
import os

import torch

from .errors import GPUOperatorNotFound

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'libbrainpylib_b200.so')
_lib = None
_targets = {}
_TARGET_TYPE = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p,
                                ctypes.c_size_t)


def lib():
  """The loaded shared library.  Missing library = hard error, never a fallback."""
  global _lib
  if _lib is None:
    if not os.path.exists(LIB_PATH):
      raise GPUOperatorNotFound('libbrainpylib_b200.so')
    _lib = ctypes.CDLL(LIB_PATH)
    _lib.bpl_last_status.restype = ctypes.c_int
    _lib.bpl_last_status.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    _lib.bpl_registration_count.restype = ctypes.c_int
    _lib.bpl_registration_name.restype = ctypes.c_char_p
    _lib.bpl_registration_name.argtypes = [ctypes.c_int]
    _lib.bpl_registration_target.restype = ctypes.c_void_p
    _lib.bpl_registration_target.argtypes = [ctypes.c_int]
    _lib.bpl_find_target.restype = ctypes.c_void_p
    _lib.bpl_find_target.argtypes = [ctypes.c_char_p]
    _lib.bpl_workspace_bytes.restype = ctypes.c_size_t
    _lib.bpl_workspace_bytes.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t]
  return _lib


def target(name):
  """ctypes callable of the custom-call target ``name``."""
  fn = _targets.get(name)
  if fn is None:
    addr = lib().bpl_find_target(name.encode())
    if not addr:   # entry points outside the reference's registry (no XLA name): plain exported symbols
      sym = getattr(lib(), name, None)
      addr = ctypes.cast(sym, ctypes.c_void_p).value if sym is not None else None
    if not addr:
      raise GPUOperatorNotFound(name)
    fn = _TARGET_TYPE(addr)
    _targets[name] = fn
  return fn


@functools.lru_cache(maxsize=4096)
def workspace_bytes(name, opaque):
  return int(lib().bpl_workspace_bytes(name.encode(), opaque, len(opaque)))


def check_status():
  buf = ctypes.create_string_buffer(256)
  code = lib().bpl_last_status(buf, 256)
  if code != 0:
    lib().bpl_clear_status()
    msg = buf.value.decode(errors='replace')
    if code == 1:
      raise RuntimeError(msg or 'Invalid opaque object size')
    raise RuntimeError(f'brainpylib_b200 kernel error ({code}): {msg}')


def call(name, buffers, opaque, device=None, stream=None):
  """Enqueue target ``name`` on ``stream`` (default: torch's current stream of ``device``).

  ``buffers``: torch CUDA tensors (operands, outputs, optional workspace) or ``None``.
  """
  if device is None:
    device = next(b.device for b in buffers if b is not None)
  if device.type != 'cuda':
    raise GPUOperatorNotFound(f'{name} (operands are on {device}, a CUDA device is required)')
  fn = target(name)
  ptrs = (ctypes.c_void_p * len(buffers))(*[None if b is None else b.data_ptr() for b in buffers])
  if stream is None:
    stream = torch.cuda.current_stream(device).cuda_stream
  if torch.cuda.current_device() == device.index:
    fn(stream, ptrs, opaque, len(opaque))
  else:
    with torch.cuda.device(device):
      fn(stream, ptrs, opaque, len(opaque))
  if _lib.bpl_last_status(None, 0) != 0:
    check_status()
