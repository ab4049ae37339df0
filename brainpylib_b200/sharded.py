"""Sharding of the transposed event-driven CSR product over the GPUs of one node.

The post-synaptic neurons (matrix columns) are cut into ``world`` contiguous ranges.  Rank ``g``
keeps, for every pre-synaptic row, only the synapses whose target lies in its range (with its own
``indptr``), and owns the same share of the neurons as spike sources.  One step is then

    1. all-gather of the spike vector (each rank contributes the spikes of its own neurons),
    2. the local product on the rank's shard -> its slice of ``y``; no reduction of ``y`` is needed.

The reference has no multi-device code at all; this layout is this library's own.
``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests) carries the exchange.
"""
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = ['column_range', 'shard_rows_by_columns', 'shard_csr_by_columns', 'ShardedEventCSR', 'PushExchange']


def column_range(n_col: int, rank: int, world: int) -> Tuple[int, int]:
  """Contiguous range of post-synaptic neurons owned by ``rank``."""
  per = (n_col + world - 1) // world
  return min(n_col, rank * per), min(n_col, (rank + 1) * per)


def shard_rows_by_columns(indices: torch.Tensor, data: Optional[torch.Tensor], row_lengths: torch.Tensor,
                          lo: int, hi: int):
  """Filter a block of complete CSR rows down to the columns ``[lo, hi)``.

  ``indices`` / ``data`` hold the rows back to back, ``row_lengths[i]`` entries each.  Returns the
  kept indices re-based to ``lo``, the kept data (``None`` for homogeneous weights) and the new
  row lengths.  Entry order inside a row is preserved.
  """
  keep = (indices >= lo) & (indices < hi)
  row_of = torch.repeat_interleave(torch.arange(row_lengths.shape[0], device=indices.device),
                                   row_lengths.to(torch.int64))
  new_lengths = torch.zeros(row_lengths.shape[0], dtype=torch.int64, device=indices.device)
  new_lengths.index_add_(0, row_of[keep], torch.ones(int(keep.sum()), dtype=torch.int64, device=indices.device))
  kept_idx = (indices[keep] - lo).to(indices.dtype)
  kept_data = None if data is None else data[keep]
  return kept_idx, kept_data, new_lengths


def shard_csr_by_columns(data: torch.Tensor, indices: torch.Tensor, indptr: torch.Tensor, n_col: int,
                         rank: int, world: int):
  """This rank's column shard of a CSR matrix: ``(data, indices, indptr, (lo, hi))``."""
  lo, hi = column_range(n_col, rank, world)
  lengths = (indptr[1:] - indptr[:-1]).to(torch.int64)
  homo = data.shape[0] == 1
  idx, dat, new_len = shard_rows_by_columns(indices, None if homo else data, lengths, lo, hi)
  ptr = torch.zeros(indptr.shape[0], dtype=torch.int64, device=indptr.device)
  ptr[1:] = torch.cumsum(new_len, 0)
  return (data if homo else dat), idx, ptr.to(indptr.dtype), (lo, hi)


class ShardedEventCSR:
  """One rank's part of ``y = A^T events`` over ``world`` ranks.

  ``local_op(data, indices, indptr, events, shape=, transpose=True)`` defaults to this library's
  CUDA operator; the CPU tests of the exchange logic pass a CPU function instead.
  """

  def __init__(self, data, indices, indptr, n_pre: int, col_range: Tuple[int, int], group=None,
               local_op: Optional[Callable] = None):
    self.data, self.indices, self.indptr = data, indices, indptr
    self.n_pre = int(n_pre)
    self.lo, self.hi = col_range
    self.group = group
    self.world = dist.get_world_size(group) if dist.is_initialized() else 1
    self.rank = dist.get_rank(group) if dist.is_initialized() else 0
    if self.n_pre % self.world != 0:
      raise ValueError('the number of pre-synaptic neurons must be divisible by the number of ranks')
    self.per = self.n_pre // self.world
    if local_op is None:
      from .event_ops import event_csr_matvec
      local_op = event_csr_matvec
    self.local_op = local_op
    self._gathered = None

  def source_range(self) -> Tuple[int, int]:
    """Pre-synaptic neurons whose spikes this rank contributes."""
    return self.rank * self.per, (self.rank + 1) * self.per

  def gather_events(self, local_events: torch.Tensor) -> torch.Tensor:
    if self.world == 1:
      return local_events
    if self._gathered is None or self._gathered.dtype != local_events.dtype or \
        self._gathered.device != local_events.device:
      self._gathered = torch.empty(self.n_pre, dtype=local_events.dtype, device=local_events.device)
    if local_events.dtype == torch.bool:   # collectives move bytes
      dist.all_gather_into_tensor(self._gathered.view(torch.uint8), local_events.contiguous().view(torch.uint8),
                                  group=self.group)
    else:
      dist.all_gather_into_tensor(self._gathered, local_events.contiguous(), group=self.group)
    return self._gathered

  def step(self, local_events: torch.Tensor) -> torch.Tensor:
    """``local_events``: the spikes of this rank's own ``n_pre / world`` source neurons.
    Returns ``y[lo:hi]``."""
    if local_events.shape[0] != self.per:
      raise ValueError(f'expected {self.per} local events, got {local_events.shape[0]}')
    events = self.gather_events(local_events)
    return self.local_op(self.data, self.indices, self.indptr, events, shape=(self.n_pre, self.hi - self.lo),
                         transpose=True)


class PushExchange:
  """All-gather of the spike vector by peer stores over NVLink instead of a collective.

  Each rank pushes its slice of the event vector into slot ``k`` of every peer's buffer
  (``bpl_spike_exchange_push``) and every rank then waits, with a bounded number of polls, until
  all slices of slot ``k`` have arrived (``bpl_spike_exchange_wait``).  The buffers live in torch
  symmetric memory so that every rank can address every peer's copy; with one rank ordinary device
  memory is used.  Kernels that follow the wait on the same stream read ``events(k)``, which is
  local memory.

  Slot discipline: call ``push`` / ``wait`` with ``k = step % slots``.  With ``slots >= 4`` a rank
  whose push of step ``s + 1`` is ordered after its own consumption of step ``s - 1`` (one step of
  run-ahead, as in ``bench.py``) can never overwrite a slot that a peer is still reading: a push
  into slot ``(s + 4) % 4`` needs this rank's step ``s + 2`` finished, which needed every peer's push
  of step ``s + 2``, which that peer ordered after its own step ``s`` finished.

  ``check()`` raises if any wait timed out (the status word is read from the device: it synchronises).
  """

  def __init__(self, n_events: int, dtype=torch.float32, device=None, group=None, slots: int = 4,
               max_polls: int = 5_000_000):
    import ctypes
    from . import _lib
    self._ctypes, self._lib = ctypes, _lib
    self.world = dist.get_world_size(group) if dist.is_initialized() else 1
    self.rank = dist.get_rank(group) if dist.is_initialized() else 0
    if n_events % self.world != 0:
      raise ValueError('the number of events must be divisible by the number of ranks')
    if self.world > 16:
      raise ValueError('at most 16 ranks')
    self.slots, self.max_polls = int(slots), int(max_polls)
    self.n_events, self.dtype = int(n_events), dtype
    self.device = torch.device('cuda', torch.cuda.current_device()) if device is None else device
    item = torch.empty(0, dtype=dtype).element_size()
    self.slice_bytes = (self.n_events // self.world) * item
    data_bytes = self.slots * self.n_events * item
    flag_words = self.slots * self.world
    lib = _lib.lib()
    lib.bpl_spike_list_slot_bytes.restype = ctypes.c_size_t
    lib.bpl_spike_list_slot_bytes.argtypes = [ctypes.c_uint32, ctypes.c_int]
    lib.bpl_spike_list_chunks_per_rank.restype = ctypes.c_uint32
    lib.bpl_spike_list_chunks_per_rank.argtypes = [ctypes.c_uint32]
    self.n_local = self.n_events // self.world
    self.list_slot_words = int(lib.bpl_spike_list_slot_bytes(self.n_local, self.world)) // 4
    self.n_chunks = int(lib.bpl_spike_list_chunks_per_rank(self.n_local)) * self.world
    data_words = (data_bytes + 3) // 4
    list_words = self.slots * self.list_slot_words
    total_words = data_words + flag_words + list_words
    if self.world == 1:
      self._buf = torch.zeros(total_words, dtype=torch.int32, device=self.device)
      bases = [self._buf.data_ptr()]
    else:
      import torch.distributed._symmetric_memory as symm_mem
      self._buf = symm_mem.empty(total_words, dtype=torch.int32, device=self.device)
      self._buf.zero_()
      self._hdl = symm_mem.rendezvous(self._buf, dist.group.WORLD if group is None else group)
      bases = [int(p) for p in self._hdl.buffer_ptrs]
      torch.cuda.synchronize()
      dist.barrier(group)      # every rank has zeroed its counters before anyone pushes
    flag_off = data_words * 4
    list_off = (data_words + flag_words) * 4
    self._peer_lists = [(ctypes.c_void_p * self.world)(*[b + list_off + k * self.list_slot_words * 4 for b in bases])
                        for k in range(self.slots)]
    self._lists = self._buf[data_words + flag_words:].view(self.slots, self.list_slot_words)
    self._peer_data = (ctypes.c_void_p * self.world)(*bases)
    self._peer_flags = (ctypes.c_void_p * self.world)(*[b + flag_off for b in bases])
    self._flags_ptr = bases[self.rank] + flag_off
    self._state = torch.zeros(self.slots + 1 + 32, dtype=torch.int32, device=self.device)
    self._data = self._buf[: data_bytes // 4].view(torch.uint8).view(dtype).view(self.slots, self.n_events)
    self._push = lib.bpl_spike_exchange_push
    self._push.restype = None
    self._push.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p,
                           ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    self._wait = lib.bpl_spike_exchange_wait
    self._wait.restype = None
    self._wait.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                           ctypes.c_uint32]

    self._push_compacted = lib.bpl_spike_exchange_push_compacted
    self._push_compacted.restype = None
    self._push_compacted.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32,
                                     ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                     ctypes.c_int, ctypes.c_int]
    self._wait_zero = lib.bpl_spike_exchange_wait_zero
    self._wait_zero.restype = None
    self._wait_zero.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                ctypes.c_int, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32]

    self._prime = lib.bpl_sharded_prime
    self._prime.restype = None
    self._prime.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32,
                            ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                            ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_uint32]
    self._step = lib.bpl_sharded_step
    self._step.restype = None
    self._step.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32,
                           ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                           ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                           ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint32]

  def _stream(self):
    return torch.cuda.current_stream(self.device).cuda_stream

  def push(self, local_events: torch.Tensor, slot: int):
    """Enqueue the push of this rank's slice (``n_events / world`` elements) into ``slot`` of every rank."""
    if local_events.dtype != self.dtype or local_events.numel() * local_events.element_size() != self.slice_bytes:
      raise ValueError('local_events must hold n_events / world elements of the exchange dtype')
    if not local_events.is_contiguous():
      local_events = local_events.contiguous()
    self._push(self._stream(), local_events.data_ptr(), self.slice_bytes, self._peer_data, self._peer_flags,
               self._state.data_ptr(), self.world, self.rank, int(slot), self.slots)
    self._lib.check_status()

  def wait(self, slot: int):
    """Enqueue the bounded wait for all slices of ``slot``."""
    self._wait(self._stream(), self._flags_ptr, self._state.data_ptr(), self.world, int(slot), self.slots,
               self.max_polls)
    self._lib.check_status()

  def push_compacted(self, local_events: torch.Tensor, slot: int):
    """Fused form: compact this rank's own events (bool or float32) and push the list of global row ids
    into ``slot`` of every rank's spike list.  Consumers then call ``wait(slot, zero=y)`` and
    ``scatter_from_list``; nobody scans the assembled vector."""
    if local_events.numel() != self.n_local or local_events.dtype not in (torch.bool, torch.uint8, torch.float32):
      raise ValueError('local_events must hold n_events / world bool or float32 elements')
    if not local_events.is_contiguous():
      local_events = local_events.contiguous()
    self._push_compacted(self._stream(), local_events.data_ptr(), int(local_events.dtype == torch.float32),
                         self.n_local, self.rank * self.n_local, self._peer_lists[int(slot)], self._peer_flags,
                         self._state.data_ptr(), self.world, self.rank, int(slot), self.slots)
    self._lib.check_status()

  def wait_zero(self, slot: int, y: torch.Tensor):
    """Bounded wait for ``slot`` and, in the same launch, zero-fill of the float32 output ``y``."""
    if y.dtype != torch.float32 or not y.is_contiguous():
      raise ValueError('y must be a contiguous float32 tensor')
    self._wait_zero(self._stream(), self._flags_ptr, self._state.data_ptr(), self.world, int(slot), self.slots,
                    self.max_polls, y.data_ptr(), y.numel())
    self._lib.check_status()

  def spike_list(self, slot: int) -> torch.Tensor:
    """The assembled spike list of ``slot`` (local memory, valid after the wait): counts, then row ids."""
    return self._lists[slot]

  def scatter_from_list(self, data, indices, indptr, slot: int, y: torch.Tensor, n_col: int):
    """``y += A^T spikes`` on this rank's shard from the list of ``slot`` (``y`` zero-filled by ``wait_zero``)."""
    from . import gpu_ops
    opaque = gpu_ops.build_triple_size_descriptor(self.n_events, n_col, self.n_chunks)
    self._lib.call('event_csr_matvec_list_heter_float', [data, indices, indptr, self._lists[slot], y], opaque,
                   device=self.device)
    return y

  # ---- one launch per step: exchange of the next step's spikes fused with this step's scatter ----
  def _check_events(self, ev):
    if ev.numel() != self.n_local or ev.dtype not in (torch.bool, torch.uint8, torch.float32):
      raise ValueError('events must hold n_events / world bool or float32 elements')
    return ev if ev.is_contiguous() else ev.contiguous()

  def prime(self, local_events: torch.Tensor, y_first: torch.Tensor):
    """Before the first ``step`` of a run: pushes this rank's spikes of that step and zero-fills its output."""
    ev = self._check_events(local_events)
    self._prime(self._stream(), ev.data_ptr(), int(ev.dtype == torch.float32), self.n_local,
                self.rank * self.n_local, self._peer_lists[0], self.list_slot_words * 4, self._peer_flags,
                self._state.data_ptr(), self.world, self.rank, self.slots, y_first.data_ptr(), y_first.numel())
    self._lib.check_status()

  def step(self, data, indices, indptr, y_cur: torch.Tensor, y_next, next_events):
    """One simulation step in one launch: ``y_cur += A_shard^T spikes(t)`` from the lists every rank pushed for
    step t, while this rank's spikes of step t + 1 (``next_events``, or None at the end of a run) go out to
    every peer and ``y_next`` (or None) is zero-filled.  ``y_cur`` must already be zero: ``prime`` clears the
    first one, every ``step`` the next.  The step counter lives on the device, so captured steps replay."""
    ev = None if next_events is None else self._check_events(next_events)
    for t in (y_cur, y_next):
      if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
        raise ValueError('outputs must be contiguous float32 tensors')
    self._step(self._stream(), data.data_ptr(), indices.data_ptr(), indptr.data_ptr(), self.n_events, y_cur.numel(),
               y_cur.data_ptr(), None if y_next is None else y_next.data_ptr(),
               None if ev is None else ev.data_ptr(), int(ev is not None and ev.dtype == torch.float32),
               self.n_local, self.rank * self.n_local, self._peer_lists[0], self.list_slot_words * 4,
               self._peer_flags, self._state.data_ptr(), self.world, self.rank, self.slots, self.max_polls)
    self._lib.check_status()
    return y_cur

  def events(self, slot: int) -> torch.Tensor:
    """The assembled event vector of ``slot`` (local memory, valid after ``wait(slot)``)."""
    return self._data[slot]

  def timed_out(self) -> bool:
    return bool(self._state[self.slots].item())

  def check(self):
    if self.timed_out():
      raise RuntimeError('spike exchange: a wait ran out of polls (a peer did not push in time); '
                         'the assembled events of that step are invalid')
