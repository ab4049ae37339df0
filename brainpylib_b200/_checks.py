"""Argument handling shared by the operator modules (torch tensors in, torch tensors out)."""
import numpy as np
import torch

_INT32_LIKE = (torch.int32, torch.uint32) if hasattr(torch, 'uint32') else (torch.int32,)


def unwrap(array):
  """brainpy arrays carry their payload in ``.value`` (brainpylib/_src/tools.py:9-13)."""
  if hasattr(array, 'is_brainpy_array') and array.is_brainpy_array:
    return array.value
  return array


def as_tensor(x, device=None, dtype=None):
  x = unwrap(x)
  if isinstance(x, torch.Tensor):
    if dtype is not None and x.dtype != dtype:
      x = x.to(dtype)
    if device is not None and x.device != device:
      x = x.to(device)
    return x
  if isinstance(x, np.ndarray) and x.dtype == np.uint32:
    x = x.view(np.int32)
  return torch.as_tensor(x, dtype=dtype, device=device)


def device_of(*arrays):
  for a in arrays:
    a = unwrap(a)
    if isinstance(a, torch.Tensor) and a.device.type == 'cuda':
      return a.device
  return torch.device('cuda', torch.cuda.current_device()) if torch.cuda.is_available() else torch.device('cpu')


def is_int32_like(t):
  return t.dtype in _INT32_LIKE


def contiguous(t):
  return t if t.is_contiguous() else t.contiguous()


def float_suffix(dtype):
  if dtype == torch.float32:
    return '_float'
  if dtype == torch.float64:
    return '_double'
  raise TypeError(f'Only support float32 and float64. But we got {dtype}.')


def loop_vmap(apply, info, in_dims, args):
  """Batching rule shared by every operator: the reference registers the same for all of its primitives
  (`register_general_batching`, brainpylib/_src/op_register/utils.py:17-38: a scan over the batch); here a Python
  loop over the batch dimension, one kernel launch per batch entry, results stacked along dimension 0."""
  outs = []
  for b in range(info.batch_size):
    # non-tensor arguments (shapes, flags, keyword dictionaries) carry a pytree of None as their in_dim
    sliced = [contiguous(a.select(d, b)) if isinstance(a, torch.Tensor) and isinstance(d, int) else a
              for a, d in zip(args, in_dims)]
    outs.append(apply(*sliced))
  return torch.stack(outs), 0
