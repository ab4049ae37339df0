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

__all__ = ['column_range', 'shard_rows_by_columns', 'shard_csr_by_columns', 'ShardedEventCSR']


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
