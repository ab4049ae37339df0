"""Exceptions of the operator layer (mirrors brainpylib/_src/errors.py:9-17)."""

__all__ = ['GPUOperatorNotFound']


class GPUOperatorNotFound(Exception):
  """Raised when the compiled CUDA library (or one of its targets) is missing.

  There is no CPU fallback: an operator either runs its CUDA kernel or raises this."""

  def __init__(self, name):
    super().__init__(
      f'GPU operator for "{name}" was not found. Build the CUDA library first: '
      f'`python -m brainpylib_b200.build` (needs nvcc; targets sm_100a).')
