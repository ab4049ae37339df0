import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)


def pytest_configure(config):
  config.addinivalue_line('markers', 'gpu: needs a CUDA device (sm_100a)')


@pytest.fixture(scope='session')
def cuda():
  import torch
  if not torch.cuda.is_available():
    pytest.skip('no CUDA device')
  return torch.device('cuda', 0)


@pytest.fixture(scope='session', autouse=True)
def _built_libraries():
  """The CUDA library and the CPU oracle are built once per session (nvcc works without a GPU)."""
  from brainpylib_b200 import build as bpl_build
  bpl_build.build()
  from oracle import cpu as oracle_cpu
  oracle_cpu.build()
