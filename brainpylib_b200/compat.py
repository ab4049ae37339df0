"""Legacy scatter operators (mirrors brainpylib/compat.py).

``csr_event_sum`` forwards to :func:`event_csr_matvec` with ``transpose=True`` exactly as
brainpylib/_src/compat/event_sum.py:66 does.  ``coo_event_sum``, ``coo_atomic_sum`` and
``coo_atomic_prod`` run the ``gpu_coo_*`` targets of the CUDA library.  ``coo_atomic_prod``
multiplies (the reference's CPU semantics, lib/cpu_atomic_prod.cc:6-43); the reference's
CUDA kernel for it adds and is not followed.
"""
import torch

from . import _lib, gpu_ops
from ._checks import as_tensor, contiguous, device_of
from .event_ops import event_csr_matvec

__all__ = ['csr_event_sum', 'coo_event_sum', 'coo_atomic_sum', 'coo_atomic_prod']


def _ftype(dtype):
  if dtype == torch.float32:
    return '_f32'
  if dtype == torch.float64:
    return '_f64'
  raise ValueError(f'The dtype of "values" must be float32 or float64, while we got {dtype}.')


def _itype(dtype):
  if dtype in (torch.int32, getattr(torch, 'uint32', torch.int32)):
    return '_i32'
  if dtype in (torch.int64, getattr(torch, 'uint64', torch.int64)):
    return '_i64'
  raise ValueError(f'The dtype of the index arrays must be integer, while we got {dtype}')


def csr_event_sum(events, pre2post, post_num, values):
  """``y[indices[j]] += values`` over the rows whose event is set (pre2post = (indices, indptr))."""
  device = device_of(events, *pre2post, values)
  events = as_tensor(events, device)
  indices, indptr = (as_tensor(a, device) for a in pre2post)
  if events.dtype != torch.bool:
    raise ValueError(f'"events" must be a vector of bool, while we got {events.dtype}')
  if len(events) + 1 != len(indptr):
    raise ValueError(f'The length of "events" must be equal to "len(pre2post[1]) - 1", '
                     f'while we get: {len(events)} + 1 != {len(indptr)}')
  if indices.dtype != indptr.dtype:
    raise ValueError(f"The dtype of pre2post[0] must be equal to that of pre2post[1], "
                     f"while we got {(indices.dtype, indptr.dtype)}")
  if indices.dtype.is_floating_point or indices.dtype == torch.bool:
    raise ValueError(f'The dtype of pre2post must be integer, while we got {indices.dtype}')
  values = torch.atleast_1d(as_tensor(values, device))
  if values.dtype not in [torch.float32, torch.float64]:
    raise ValueError(f'The dtype of "values" must be float32 or float64, while we got {values.dtype}.')
  if values.numel() not in [1, indices.numel()]:
    raise ValueError(f'The size of "values" must be 1 (a scalar) or len(pre2post[0]) (a vector), '
                     f'while we got {values.numel()} != 1 != {indices.numel()}')
  if indices.dtype == torch.int64:
    indices, indptr = indices.to(torch.int32), indptr.to(torch.int32)
  return event_csr_matvec(values, indices, indptr, events, shape=(events.shape[0], int(post_num)), transpose=True)


def coo_event_sum(events, pre_ids, post_ids, post_num, values):
  """``if events[pre_ids[i]]: y[post_ids[i]] += values[i]`` (lib/gpu_event_sum.cu:122-206)."""
  device = device_of(events, pre_ids, post_ids, values)
  events = contiguous(as_tensor(events, device))
  pre_ids, post_ids = contiguous(as_tensor(pre_ids, device)), contiguous(as_tensor(post_ids, device))
  if events.dtype != torch.bool:
    raise ValueError(f'"events" must be a vector of bool, while we got {events.dtype}')
  if pre_ids.shape != post_ids.shape or pre_ids.dtype != post_ids.dtype:
    raise ValueError('pre_ids and post_ids must have the same shape and dtype')
  values = contiguous(torch.atleast_1d(as_tensor(values, device)))
  if values.numel() not in [1, pre_ids.numel()]:
    raise ValueError(f'The size of "values" must be 1 (a scalar) or len(pre_ids) (a vector), '
                     f'while we got {values.numel()} != 1 != {pre_ids.numel()}')
  homo = '_homo' if values.numel() == 1 else '_heter'
  name = 'gpu_coo_event_sum' + homo + _ftype(values.dtype) + _itype(pre_ids.dtype)
  out = torch.empty(int(post_num), dtype=values.dtype, device=device)
  opaque = gpu_ops.build_coo_event_sum_descriptor(pre_ids.numel(), int(post_num))
  _lib.call(name, [events, pre_ids, post_ids, values, out], opaque, device=device)
  return out


def _coo_atomic(op, values, post_ids, post_num, pre_ids):
  device = device_of(values, post_ids, pre_ids)
  values = contiguous(torch.atleast_1d(as_tensor(values, device)))
  post_ids = contiguous(as_tensor(post_ids, device))
  out = torch.empty(int(post_num), dtype=values.dtype, device=device)
  build = gpu_ops.build_coo_atomic_sum_descriptor if op == 'sum' else gpu_ops.build_coo_atomic_prod_descriptor
  opaque = build(post_ids.numel(), int(post_num))
  if values.numel() == 1:
    name = f'gpu_coo_atomic_{op}_homo' + _ftype(values.dtype) + _itype(post_ids.dtype)
    _lib.call(name, [values, post_ids, out], opaque, device=device)
  else:
    if pre_ids is None:
      raise ValueError('"pre_ids" must be provided when "values" is a vector')
    pre_ids = contiguous(as_tensor(pre_ids, device))
    if pre_ids.shape != post_ids.shape or pre_ids.dtype != post_ids.dtype:
      raise ValueError('pre_ids and post_ids must have the same shape and dtype')
    if pre_ids.dtype.is_floating_point or pre_ids.dtype == torch.bool:
      raise ValueError(f'The dtype of post_ids must be a subtype of integer, while we got {post_ids.dtype}')
    # the kernel reads values[pre_ids[i]]: the reference's host check (brainpylib/_src/compat/atomic_sum.py:54-56)
    # keeps a bad id from becoming an out-of-bounds read on the device (one reduction + host read of a scalar)
    if pre_ids.numel() and (values.numel() <= int(pre_ids.max()) or int(pre_ids.min()) < 0):
      raise ValueError(f'The size of "values" must be 1 (a scalar) or longer than pre_size (a vector), '
                       f'while we got {values.numel()} != 1 <= {int(pre_ids.max())}')
    name = f'gpu_coo_atomic_{op}_heter' + _ftype(values.dtype) + _itype(post_ids.dtype)
    _lib.call(name, [values, pre_ids, post_ids, out], opaque, device=device)
  return out


def coo_atomic_sum(values, post_ids, post_num, pre_ids=None):
  """``y[post_ids[i]] += values[pre_ids[i]]`` (scalar ``values``: ``+= values``)."""
  return _coo_atomic('sum', values, post_ids, post_num, pre_ids)


def coo_atomic_prod(values, post_ids, post_num, pre_ids=None):
  """``y[post_ids[i]] *= values[pre_ids[i]]`` starting from 1 (scalar ``values``: ``*= values``)."""
  return _coo_atomic('prod', values, post_ids, post_num, pre_ids)
