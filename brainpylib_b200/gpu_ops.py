"""The module the reference imports as ``from brainpylib import gpu_ops``
(lib/gpu_ops.cc): ``registrations()`` maps every XLA custom-call target name to a
``PyCapsule`` named ``"xla._CUSTOM_CALL_TARGET"``, and the ``build_*_descriptor``
functions return the packed opaque bytes.  Here it is a thin layer over the C ABI of
``libbrainpylib_b200.so`` (no pybind11 module is needed).
"""
import ctypes
import functools

from . import _lib

__all__ = [
  'registrations', 'target_names', 'register_custom_call_targets',
  'build_twouint_onebool_descriptor', 'build_double_size_descriptor', 'build_triple_size_descriptor',
  'build_jitconn_prob_homo_descriptor', 'build_jitconn_prob_uniform_descriptor',
  'build_jitconn_prob_normal_descriptor', 'build_matmat_jit_prob_descriptor1',
  'build_csr_event_sum_descriptor', 'build_coo_event_sum_descriptor',
  'build_coo_atomic_sum_descriptor', 'build_coo_atomic_prod_descriptor', 'build_nonzero_descriptor',
]

_CAPSULE_NAME = b'xla._CUSTOM_CALL_TARGET'   # lib/pybind11_kernel_helpers.h:20-23


def target_names():
  lib = _lib.lib()
  return [lib.bpl_registration_name(i).decode() for i in range(lib.bpl_registration_count())]


def registrations():
  """``{target name: PyCapsule("xla._CUSTOM_CALL_TARGET")}`` (lib/gpu_ops.cc:24-177)."""
  lib = _lib.lib()
  new_capsule = ctypes.pythonapi.PyCapsule_New
  new_capsule.restype = ctypes.py_object
  new_capsule.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p]
  out = {}
  for i in range(lib.bpl_registration_count()):
    out[lib.bpl_registration_name(i).decode()] = new_capsule(lib.bpl_registration_target(i), _CAPSULE_NAME, None)
  return out


def register_custom_call_targets(xla_client=None, platform='gpu'):
  """Registers every target with XLA, as the reference does at import time
  (brainpylib/_src/register_custom_calls.py:16-22).  ``xla_client`` defaults to ``jax.lib.xla_client``;
  without JAX installed the import error propagates (there is nothing to register with).  Returns the
  registered names."""
  if xla_client is None:
    from jax.lib import xla_client
  names = []
  for name, capsule in registrations().items():
    xla_client.register_custom_call_target(name, capsule, platform=platform)
    names.append(name)
  return names


@functools.lru_cache(maxsize=4096)
def _build(fn_name, argtypes, args):
  fn = getattr(_lib.lib(), fn_name)
  fn.restype = ctypes.c_size_t
  fn.argtypes = list(argtypes) + [ctypes.c_void_p, ctypes.c_size_t]   # descriptors are pure functions of their arguments: cached
  buf = ctypes.create_string_buffer(64)
  n = fn(*args, buf, 64)
  if n == 0:
    raise RuntimeError(f'{fn_name} failed')
  return buf.raw[:n]


_U, _F, _I = ctypes.c_uint32, ctypes.c_float, ctypes.c_int


def _u32(x):
  return int(x) & 0xffffffff


def build_twouint_onebool_descriptor(uint_x, uint_y, bool_x):
  return _build('bpl_build_twouint_onebool_descriptor', (_U, _U, _I), (_u32(uint_x), _u32(uint_y), int(bool(bool_x))))


def build_double_size_descriptor(size_x, size_y):
  return _build('bpl_build_double_size_descriptor', (_U, _U), (_u32(size_x), _u32(size_y)))


def build_triple_size_descriptor(size_x, size_y, size_z):
  return _build('bpl_build_triple_size_descriptor', (_U, _U, _U), (_u32(size_x), _u32(size_y), _u32(size_z)))


def build_jitconn_prob_homo_descriptor(n_row, n_col, seed, prob):
  return _build('bpl_build_jitconn_prob_homo_descriptor', (_U, _U, _U, _F),
                (_u32(n_row), _u32(n_col), _u32(seed), float(prob)))


def build_jitconn_prob_uniform_descriptor(n_row, n_col, seed, prob, w_min, w_range):
  return _build('bpl_build_jitconn_prob_uniform_descriptor', (_U, _U, _U, _F, _F, _F),
                (_u32(n_row), _u32(n_col), _u32(seed), float(prob), float(w_min), float(w_range)))


def build_jitconn_prob_normal_descriptor(n_row, n_col, seed, prob, w_mu, w_sigma):
  return _build('bpl_build_jitconn_prob_normal_descriptor', (_U, _U, _U, _F, _F, _F),
                (_u32(n_row), _u32(n_col), _u32(seed), float(prob), float(w_mu), float(w_sigma)))


def build_matmat_jit_prob_descriptor1(m, k, n, seed, log_p, w1, w2):
  return _build('bpl_build_matmat_jit_prob_descriptor1', (_U, _U, _U, _U, _F, _F, _F),
                (_u32(m), _u32(k), _u32(n), _u32(seed), float(log_p), float(w1), float(w2)))


def _two(name):
  def build(size_x, size_y):
    return _build(name, (_U, _U), (_u32(size_x), _u32(size_y)))
  build.__name__ = name[4:]
  return build


build_csr_event_sum_descriptor = _two('bpl_build_csr_event_sum_descriptor')
build_coo_event_sum_descriptor = _two('bpl_build_coo_event_sum_descriptor')
build_coo_atomic_sum_descriptor = _two('bpl_build_coo_atomic_sum_descriptor')
build_coo_atomic_prod_descriptor = _two('bpl_build_coo_atomic_prod_descriptor')
build_nonzero_descriptor = _two('bpl_build_nonzero_descriptor')
