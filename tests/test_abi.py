"""Host-side checks of the C ABI: the library loads, exports every symbol the public
header declares, packs descriptors byte-identically to the reference's structs
(lib/kernel_helper_descriptor.cuh:49-144), and reports errors without raising across the
boundary.  No kernel is launched here."""
import ctypes
import os
import re
import struct
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, 'include', 'brainpylib_b200.h')


def declared_symbols():
  """Function names declared in the header, with the target list macro expanded by the preprocessor."""
  text = ''.join(line for line in open(HEADER) if not line.lstrip().startswith('#include'))
  out = subprocess.run(['gcc', '-E', '-P', '-x', 'c', '-'], input=text, check=True, capture_output=True,
                       text=True).stdout
  names = re.findall(r'\b(\w+)\s*\([^;{()]*\)\s*;', out)
  return sorted(set(names))


def test_library_exports_every_declared_symbol():
  from brainpylib_b200 import _lib
  lib = _lib.lib()
  names = declared_symbols()
  assert len(names) > 100
  for n in names:
    if n == 'bpl_custom_call_t':
      continue
    assert hasattr(lib, n), f'{n} is declared in include/brainpylib_b200.h but not exported'


def test_registrations_are_xla_capsules():
  from brainpylib_b200 import gpu_ops
  regs = gpu_ops.registrations()
  assert len(regs) == len(gpu_ops.target_names()) == 129
  get_name = ctypes.pythonapi.PyCapsule_GetName
  get_name.restype = ctypes.c_char_p
  get_name.argtypes = [ctypes.py_object]
  get_ptr = ctypes.pythonapi.PyCapsule_GetPointer
  get_ptr.restype = ctypes.c_void_p
  get_ptr.argtypes = [ctypes.py_object, ctypes.c_char_p]
  for name, capsule in regs.items():
    assert get_name(capsule) == b'xla._CUSTOM_CALL_TARGET'
    assert get_ptr(capsule, b'xla._CUSTOM_CALL_TARGET')
  # the names the reference's Python layer asks for (lib/gpu_ops.cc:79-174)
  for n in ['event_csr_matvec_homo_float_bool', 'event_csr_matvec_heter_double_double',
            'csr_matvec_heter_vector_float', 'csr_matvec_homo_adaptive_double',
            'gpu_event_matvec_prob_uniform_v2_float_bool', 'gpu_event_matvec_atomic_prob_normal_v2_double_double',
            'gpu_matvec_prob_homo_v2_float', 'gpu_matvec_atomic_prob_normal_v2_double',
            'gpu_matmat_prob_prob_normal_float_v1', 'gpu_matmat_prob_prob_uniform_double_v1',
            'gpu_csr_event_sum_homo_f32_i32', 'gpu_coo_event_sum_heter_f64_i64',
            'gpu_coo_atomic_sum_heter_f32_i32', 'gpu_coo_atomic_prod_homo_f64_i64']:
    assert n in regs, n


def test_descriptor_layouts():
  from brainpylib_b200 import gpu_ops as g
  d = g.build_twouint_onebool_descriptor(7, 9, True)
  assert len(d) == 12 and struct.unpack('<II?3x', d) == (7, 9, True)
  d = g.build_double_size_descriptor(5, 6)
  assert len(d) == 8 and struct.unpack('<II', d) == (5, 6)
  p = float(np.log(1 - 0.001))
  d = g.build_jitconn_prob_homo_descriptor(10, 20, 42, p)
  assert len(d) == 24
  n_row, n_col, seed, prob = struct.unpack('<III4xd', d)
  assert (n_row, n_col, seed) == (10, 20, 42)
  # the builder takes a float: the double field holds the float32-rounded value
  assert prob == float(np.float32(p)) and prob != p
  for build in (g.build_jitconn_prob_uniform_descriptor, g.build_jitconn_prob_normal_descriptor):
    d = build(1, 2, 3, p, -0.1, 0.2)
    assert len(d) == 40
    assert struct.unpack('<III4xddd', d) == (1, 2, 3, float(np.float32(p)), float(np.float32(-0.1)),
                                             float(np.float32(0.2)))
  d = g.build_matmat_jit_prob_descriptor1(256, 65536, 65536, 7, p, 0., 0.01)
  assert len(d) == 40
  assert struct.unpack('<IIIIddd', d) == (256, 65536, 65536, 7, float(np.float32(p)), 0., float(np.float32(0.01)))
  for build in (g.build_csr_event_sum_descriptor, g.build_coo_event_sum_descriptor,
                g.build_coo_atomic_sum_descriptor, g.build_coo_atomic_prod_descriptor, g.build_nonzero_descriptor):
    assert struct.unpack('<II', build(11, 12)) == (11, 12)
  # seeds wrap to 32 bits like the reference's `unsigned int` parameter
  assert struct.unpack('<III4xd', g.build_jitconn_prob_homo_descriptor(1, 1, 2 ** 32 + 5, 0.))[2] == 5


def test_wrong_opaque_size_sets_status_and_launches_nothing():
  """The reference throws std::runtime_error("Invalid opaque object size") (lib/kernel_helpers.h:36-38);
  here the call returns and the status says so.  The size check precedes any CUDA call."""
  from brainpylib_b200 import _lib
  lib = _lib.lib()
  lib.bpl_clear_status()
  fn = _lib.target('event_csr_matvec_homo_float_bool')
  bufs = (ctypes.c_void_p * 6)()
  fn(None, bufs, b'\x00' * 5, 5)
  msg = ctypes.create_string_buffer(256)
  assert lib.bpl_last_status(msg, 256) == 1
  assert msg.value == b'Invalid opaque object size'
  with pytest.raises(RuntimeError, match='Invalid opaque object size'):
    _lib.check_status()
  assert lib.bpl_last_status(None, 0) == 0
  for name in ('csr_matvec_heter_vector_float', 'gpu_matvec_prob_homo_v2_float',
               'gpu_event_matvec_prob_normal_v2_float_bool', 'gpu_matmat_prob_prob_normal_float_v1',
               'gpu_coo_atomic_sum_homo_f32_i32'):
    _lib.target(name)(None, bufs, b'', 0)
    assert lib.bpl_last_status(None, 0) == 1
    lib.bpl_clear_status()


def test_workspace_query():
  from brainpylib_b200 import _lib, gpu_ops
  t = gpu_ops.build_twouint_onebool_descriptor(1_000_000, 1_000_000, True)
  f = gpu_ops.build_twouint_onebool_descriptor(1_000_000, 1_000_000, False)
  assert _lib.workspace_bytes('event_csr_matvec_heter_float_float', t) == (1024 + 1_000_000) * 4
  assert _lib.workspace_bytes('event_csr_matvec_heter_float_float', f) == 0
  assert _lib.workspace_bytes('csr_matvec_heter_vector_float', gpu_ops.build_double_size_descriptor(3, 4)) == 0


def test_unknown_target_and_cpu_tensors_fail_loudly():
  import torch
  import brainpylib_b200 as b
  from brainpylib_b200 import _lib
  with pytest.raises(b.GPUOperatorNotFound):
    _lib.target('no_such_target')
  if not torch.cuda.is_available():
    with pytest.raises(b.GPUOperatorNotFound):   # no CPU fallback
      b.event_csr_matvec(0.6, torch.zeros(3, dtype=torch.int32), torch.tensor([0, 1, 3], dtype=torch.int32),
                         torch.tensor([True, False]), shape=(2, 4), transpose=True)
    with pytest.raises(b.GPUOperatorNotFound):
      b.matvec_prob_conn_homo_weight(torch.zeros(4), 1., conn_prob=0.1, shape=(2, 4), seed=1)


def test_argument_checks_match_reference():
  """Errors raised before any device work (brainpylib/_src/event_ops/event_csr_matvec.py:75-99,
  brainpylib/_src/sparse_ops/sparse_csr_matvec.py:71-83, brainpylib/_src/jitconn_ops/matmat.py:171-174)."""
  import torch
  import brainpylib_b200 as b
  idx = torch.zeros(3, dtype=torch.int32)
  ptr = torch.tensor([0, 1, 3], dtype=torch.int32)
  with pytest.raises(ValueError, match='size of data'):
    b.event_csr_matvec(torch.zeros(2), idx, ptr, torch.zeros(2, dtype=torch.bool), shape=(2, 4), transpose=True)
  with pytest.raises(ValueError, match='int32 or uint32'):
    b.event_csr_matvec(1., idx.to(torch.int64), ptr, torch.zeros(2, dtype=torch.bool), shape=(2, 4), transpose=True)
  with pytest.raises(ValueError, match='Shape mismatch, vec'):
    b.event_csr_matvec(1., idx, ptr, torch.zeros(4, dtype=torch.bool), shape=(2, 4), transpose=True)
  with pytest.raises(ValueError, match='Shape mismatch, mat'):
    b.event_csr_matvec(1., idx, ptr, torch.zeros(2, dtype=torch.bool), shape=(2, 4), transpose=False)
  with pytest.raises(ValueError, match='Only support methods'):
    b.csr_matvec(torch.zeros(3), idx, ptr, torch.zeros(4), shape=(2, 4), method='fancy')
  with pytest.raises(TypeError, match='types of data and vector'):
    b.csr_matvec(torch.zeros(3), idx, ptr, torch.zeros(4, dtype=torch.float64), shape=(2, 4))
  with pytest.raises(ValueError, match='Seed cannot be none'):
    b.matmat_prob_conn_normal_weight(torch.zeros(2, 4), w_mu=0., w_sigma=1., conn_prob=0.1, shape=(4, 5))
  with pytest.raises(ValueError, match='Shape mismatch, X'):
    b.matmat_prob_conn_normal_weight(torch.zeros(2, 3), w_mu=0., w_sigma=1., conn_prob=0.1, shape=(4, 5), seed=1)
  with pytest.raises(ValueError, match='1D vector'):
    b.event_matvec_prob_conn_homo_weight(torch.zeros(2, 2), 1., conn_prob=0.1, shape=(2, 2), seed=1)


def test_registration_with_xla_through_a_stand_in_client():
  """register_custom_call_targets hands every target to the client the way the reference's import-time loop
  does (brainpylib/_src/register_custom_calls.py:16-22): name, capsule "xla._CUSTOM_CALL_TARGET", platform gpu."""
  from brainpylib_b200 import _lib, gpu_ops

  class Client:
    def __init__(self):
      self.seen = []

    def register_custom_call_target(self, name, capsule, platform):
      self.seen.append((name, capsule, platform))

  client = Client()
  names = gpu_ops.register_custom_call_targets(client)
  assert names == gpu_ops.target_names() and len(client.seen) == len(names)
  get_name = ctypes.pythonapi.PyCapsule_GetName
  get_name.restype, get_name.argtypes = ctypes.c_char_p, [ctypes.py_object]
  get_ptr = ctypes.pythonapi.PyCapsule_GetPointer
  get_ptr.restype, get_ptr.argtypes = ctypes.c_void_p, [ctypes.py_object, ctypes.c_char_p]
  lib = _lib.lib()
  for name, capsule, platform in client.seen:
    assert platform == 'gpu'
    assert get_name(capsule) == b'xla._CUSTOM_CALL_TARGET'
    assert get_ptr(capsule, b'xla._CUSTOM_CALL_TARGET') == ctypes.cast(lib.bpl_find_target(name.encode()), ctypes.c_void_p).value


def test_sharded_step_refuses_bad_arguments_before_any_launch():
  """Argument checks of the one-launch step entry points run on the host and report through the status channel
  (fewer than four slots cannot keep a slow peer's list from being overwritten; null tables cannot be launched)."""
  from brainpylib_b200 import _lib
  lib = _lib.lib()
  vp, u32, i32 = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_int
  lib.bpl_sharded_step.restype = None
  lib.bpl_sharded_step.argtypes = [vp] * 4 + [u32, u32] + [vp] * 3 + [i32, u32, u32, vp, ctypes.c_size_t, vp, vp,
                                                                  i32, i32, i32, u32]
  state = ctypes.create_string_buffer(4 * 64)
  msg = ctypes.create_string_buffer(256)

  def step(slots, world=1, rank=0, n_local=10):
    lib.bpl_clear_status()
    lib.bpl_sharded_step(None, None, None, None, 10, 10, None, None, None, 0, n_local, 0, None, 1024, None,
                         ctypes.cast(state, vp), world, rank, slots, 10)
    return lib.bpl_last_status(msg, 256), msg.value.decode()

  code, text = step(slots=3)
  assert code == 3 and 'slots >= 4' in text
  code, text = step(slots=4, world=17)
  assert code == 3 and 'world 1..16' in text
  code, text = step(slots=4, n_local=5_000_000)          # 1221 chunks of 4096 events: beyond the 1024 of a list
  assert code == 3 and '1024 chunks' in text
  code, text = step(slots=4)
  assert code == 3 and 'null' in text
  lib.bpl_clear_status()


def test_host_step_runs_refuse_bad_arguments_before_any_launch():
  """bpl_run_host_steps / bpl_sharded_run_host_steps check their arguments on the host: unknown target, group outside
  1..16, missing ring buffers, streams that are not distinct."""
  from brainpylib_b200 import _lib
  lib = _lib.lib()
  vp, u32, i32, sz = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_int, ctypes.c_size_t
  run = lib.bpl_run_host_steps
  run.restype = None
  run.argtypes = [ctypes.c_char_p, ctypes.c_char_p, sz, vp, i32, i32, i32, i32, vp, vp, vp, u32, vp, sz, vp, sz, u32, u32,
                  vp, vp, vp]
  msg = ctypes.create_string_buffer(256)
  opaque = b'\0' * 12
  bufs = (vp * 6)(*[0x1000 + 256 * i for i in range(6)])          # never dereferenced by the checks
  ring3 = (vp * 3)(0x9000, 0xa000, 0xb000)
  host = ctypes.create_string_buffer(64)

  def call(name=b'event_csr_matvec_heter_float_float', group=1, in_ring=ring3, streams=(0x10, 0x20, 0x30), n_buffers=6):
    lib.bpl_clear_status()
    run(name, opaque, 12, bufs, n_buffers, 3, 4, 5, in_ring, ring3, ring3, group, ctypes.cast(host, vp), 16,
        ctypes.cast(host, vp), 16, 1, 4, *streams)
    return lib.bpl_last_status(msg, 256), msg.value.decode()

  assert call(name=b'no_such_target') == (3, 'host steps: unknown target')
  code, text = call(group=0)
  assert code == 3 and 'group' in text
  code, text = call(group=17)
  assert code == 3 and 'group' in text
  code, text = call(in_ring=(vp * 3)(0x9000, None, 0xb000))
  assert code == 3 and 'null buffer' in text
  code, text = call(streams=(0x10, 0x10, 0x30))
  assert code == 3 and 'distinct' in text
  code, text = call(n_buffers=3)
  assert code == 3 and 'out of range' in text

  srun = lib.bpl_sharded_run_host_steps
  srun.restype = None
  srun.argtypes = [vp, vp, u32, u32, i32, i32, u32, i32, u32, u32, vp, sz, vp, vp, i32, i32, i32, u32, vp, vp, u32, vp, vp,
                   u32, u32, vp, vp, vp]
  ring4 = (vp * 4)(0x9000, 0xa000, 0xb000, 0xc000)

  def scall(group=1, ev_ring=ring4, streams=(0x10, 0x20, 0x30)):
    lib.bpl_clear_status()
    srun(0x1000, 0x2000, 10, 32, 0, 0, 2, 1, 10, 0, None, 1024, None, None, 1, 0, 4, 10, ev_ring, ring3, group,
         ctypes.cast(host, vp), ctypes.cast(host, vp), 1, 4, *streams)
    return lib.bpl_last_status(msg, 256), msg.value.decode()

  code, text = scall(group=0)
  assert code == 3 and 'group' in text
  code, text = scall(ev_ring=(vp * 4)(0x9000, 0xa000, 0xb000, None))      # the buffer of step 0 is missing
  assert code == 3 and 'null buffer' in text
  code, text = scall(streams=(0x10, 0x20, 0x20))
  assert code == 3 and 'distinct' in text
  lib.bpl_clear_status()
