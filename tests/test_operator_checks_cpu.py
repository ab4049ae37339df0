"""Host side of the operator layer, without a GPU: the public names of the reference's operators for this path
exist, argument checks raise what the reference raises (same error types and messages,
brainpylib/_src/event_ops/event_csr_matvec.py, _src/sparse_ops/sparse_csr_matvec.py, _src/jitconn_ops/matvec.py:
88-102,177-187), and operands on the CPU are refused with GPUOperatorNotFound: there is no CPU fallback."""
import pytest
import torch

import brainpylib_b200 as bpl
from brainpylib_b200 import jitconn_ops


def _csr():
  d = torch.ones(3)
  i = torch.tensor([0, 1, 2], dtype=torch.int32)
  p = torch.tensor([0, 1, 2, 3], dtype=torch.int32)
  return d, i, p


def test_public_names_of_the_reference_operators_exist():
  for name in ('event_csr_matvec', 'csr_matvec', 'cusparse_csr_matvec', 'event_info',
               'matvec_prob_conn_homo_weight', 'matvec_prob_conn_uniform_weight', 'matvec_prob_conn_normal_weight',
               'event_matvec_prob_conn_homo_weight', 'event_matvec_prob_conn_uniform_weight',
               'event_matvec_prob_conn_normal_weight', 'matmat_prob_conn_uniform_weight',
               'matmat_prob_conn_normal_weight', 'coo_atomic_sum', 'coo_atomic_prod', 'coo_event_sum',
               'csr_event_sum', 'GPUOperatorNotFound'):
    assert hasattr(bpl, name), name


def test_operands_on_the_cpu_are_refused_not_computed():
  d, i, p = _csr()
  with pytest.raises(bpl.GPUOperatorNotFound):
    bpl.event_csr_matvec(d, i, p, torch.ones(3, dtype=torch.bool), shape=(3, 3), transpose=True)
  with pytest.raises(bpl.GPUOperatorNotFound):
    bpl.csr_matvec(d, i, p, torch.ones(3), shape=(3, 3))
  with pytest.raises(bpl.GPUOperatorNotFound):
    bpl.event_matvec_prob_conn_homo_weight(torch.ones(3, dtype=torch.bool), 1.0, conn_prob=0.1, shape=(3, 3), seed=1)
  with pytest.raises(bpl.GPUOperatorNotFound):
    bpl.matvec_prob_conn_uniform_weight(torch.ones(3), w_low=0., w_high=1., conn_prob=0.1, shape=(3, 3), seed=1)
  with pytest.raises(bpl.GPUOperatorNotFound):
    bpl.matmat_prob_conn_normal_weight(torch.ones(2, 3), w_mu=0., w_sigma=1., conn_prob=0.1, shape=(3, 3), seed=1)


def test_shape_checks_raise_the_reference_messages():
  d, i, p = _csr()
  with pytest.raises(ValueError, match=r'Shape mismatch, vec \(4,\) @ mat \(3, 3\)\.'):
    bpl.event_csr_matvec(d, i, p, torch.ones(4, dtype=torch.bool), shape=(3, 3), transpose=True)
  with pytest.raises(ValueError, match=r'Shape mismatch, mat \(3, 5\) @ vec \(4,\)\.'):
    bpl.matvec_prob_conn_homo_weight(torch.ones(4), 1.0, conn_prob=0.1, shape=(3, 5), seed=1)
  with pytest.raises(ValueError, match=r'Shape mismatch, vec \(4,\) @ mat \(3, 5\)\.'):
    bpl.matvec_prob_conn_homo_weight(torch.ones(4), 1.0, conn_prob=0.1, shape=(3, 5), seed=1, transpose=True)
  with pytest.raises(ValueError, match='should be a 1D vector'):
    bpl.matvec_prob_conn_normal_weight(torch.ones(4, 2), w_mu=0., w_sigma=1., conn_prob=0.1, shape=(3, 4), seed=1)
  with pytest.raises(ValueError, match='length-2 tuple'):
    bpl.event_matvec_prob_conn_homo_weight(torch.ones(4, dtype=torch.bool), 1.0, conn_prob=0.1, shape=(3, 4, 5), seed=1)
  with pytest.raises(AssertionError):
    bpl.matvec_prob_conn_uniform_weight(torch.ones(4), w_low=1., w_high=0., conn_prob=0.1, shape=(3, 4), seed=1)


def test_versions_the_reference_does_not_register_are_refused():
  """lib/gpu_ops.cc:166-174: normal weights have v1, v2 and v3, uniform weights v1 only."""
  with pytest.raises(ValueError, match="version must be 'v1'"):
    bpl.matmat_prob_conn_uniform_weight(torch.ones(2, 3), w_low=0., w_high=1., conn_prob=0.1, shape=(3, 3), seed=1,
                                        version='v2')
  with pytest.raises(ValueError, match="version must be 'v1'"):
    bpl.matmat_prob_conn_normal_weight(torch.ones(2, 3), w_mu=0., w_sigma=1., conn_prob=0.1, shape=(3, 3), seed=1,
                                       version='v4')
  with pytest.raises(AssertionError):
    bpl.matvec_prob_conn_homo_weight(torch.ones(3), 1.0, conn_prob=0.1, shape=(3, 3), seed=1, version='v3')


def test_coo_atomic_refuses_a_pre_id_beyond_values_before_any_launch():
  """The reference's host check (brainpylib/_src/compat/atomic_sum.py:54-56): without it the kernel would read
  values[pre_ids[i]] out of bounds on the device."""
  import torch
  import pytest
  from brainpylib_b200 import compat
  values = torch.ones(4)
  post = torch.tensor([0, 1, 2], dtype=torch.int32)
  for bad in (torch.tensor([0, 4, 1], dtype=torch.int32), torch.tensor([0, -1, 1], dtype=torch.int32)):
    with pytest.raises(ValueError, match='longer than pre_size'):
      compat.coo_atomic_sum(values, post, 3, pre_ids=bad)
    with pytest.raises(ValueError, match='longer than pre_size'):
      compat.coo_atomic_prod(values, post, 3, pre_ids=bad)
