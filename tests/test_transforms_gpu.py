"""Batching (`torch.func.vmap`) and forward-mode differentiation (`torch.func.jvp`) of the operators: the rules the
reference registers for its primitives (batching for all of them through `register_general_batching`,
brainpylib/_src/op_register/utils.py:17-38; JVPs at event_csr_matvec.py:439-444, cusparse_matvec.py:281-286,
matvec.py:371-390, event_matvec.py:242-260).  The batched calls mirror the reference's own tests
(brainpylib/_src/event_ops/tests/test_event_csr_matvec.py:94-129, jitconn_ops/tests/test_event_matvec.py:139-147,
matmat_testcase.py:59-78): vmap over data, over events, over both == a Python loop."""
import numpy as np
import pytest
import torch
from torch.func import jvp, vmap

import cases
import brainpylib_b200 as bpl

pytestmark = pytest.mark.gpu


def _csr(cuda, shape, prob, seed):
  data, indices, indptr, rng = cases.csr_case(shape, prob, seed)
  return [torch.as_tensor(a).to(cuda) for a in (data, indices, indptr)], rng


@pytest.mark.parametrize('transpose', [True, False])
@pytest.mark.parametrize('shape', [(100, 200), (200, 100), (10, 1000)])
def test_event_csr_matvec_vmap_over_data_events_and_both(cuda, shape, transpose):
  (data, indices, indptr), rng = _csr(cuda, shape, 0.3, 51)
  n_in = shape[0] if transpose else shape[1]
  B = 5
  events = torch.as_tensor(rng.random((B, n_in)) < 0.2).to(cuda)
  datas = torch.as_tensor(rng.standard_normal((B, data.shape[0])).astype(np.float32)).to(cuda)
  op = lambda d, e: bpl.event_csr_matvec(d, indices, indptr, e, shape=shape, transpose=transpose)
  tol = dict(rtol=1e-5, atol=1e-4)
  torch.testing.assert_close(vmap(lambda e: op(data, e))(events), torch.stack([op(data, events[b]) for b in range(B)]), **tol)
  torch.testing.assert_close(vmap(lambda d: op(d, events[0]))(datas), torch.stack([op(datas[b], events[0]) for b in range(B)]), **tol)
  torch.testing.assert_close(vmap(op)(datas, events), torch.stack([op(datas[b], events[b]) for b in range(B)]), **tol)
  # batch dimension 1 for the events, homogeneous weight
  homo = torch.tensor([1.5], device=cuda)
  got = vmap(lambda e: bpl.event_csr_matvec(homo, indices, indptr, e, shape=shape, transpose=transpose), in_dims=1)(events.T.contiguous())
  want = torch.stack([bpl.event_csr_matvec(homo, indices, indptr, events[b], shape=shape, transpose=transpose) for b in range(B)])
  assert torch.equal(got, want)


@pytest.mark.parametrize('transpose', [True, False])
def test_event_csr_matvec_jvp_matches_dense_algebra(cuda, transpose):
  shape = (120, 90)
  (data, indices, indptr), rng = _csr(cuda, shape, 0.3, 52)
  dense = bpl.csr_to_dense(data, indices, indptr, shape=shape).double()
  n_in = shape[0] if transpose else shape[1]
  ev = torch.as_tensor((rng.random(n_in) < 0.3).astype(np.float32)).to(cuda)
  d_dot = torch.as_tensor(rng.standard_normal(data.shape[0]).astype(np.float32)).to(cuda)
  e_dot = torch.as_tensor(rng.standard_normal(n_in).astype(np.float32)).to(cuda)
  f = lambda d, e: bpl.event_csr_matvec(d, indices, indptr, e, shape=shape, transpose=transpose)
  primal, tangent = jvp(f, (data, ev), (d_dot, e_dot))
  dense_dot = bpl.csr_to_dense(d_dot, indices, indptr, shape=shape).double()
  mv = (lambda m, v: v.double() @ m) if transpose else (lambda m, v: m @ v.double())
  torch.testing.assert_close(primal.double(), mv(dense, ev), rtol=1e-5, atol=1e-4)
  # data tangent: the event product of data_dot; events tangent: the DENSE product with events_dot (the reference's rule)
  torch.testing.assert_close(tangent.double(), mv(dense_dot, ev) + mv(dense, e_dot), rtol=1e-4, atol=1e-3)


def test_csr_matvec_vmap_and_jvp(cuda):
  shape = (150, 80)
  (data, indices, indptr), rng = _csr(cuda, shape, 0.2, 53)
  dense = bpl.csr_to_dense(data, indices, indptr, shape=shape).double()
  for transpose in (False, True):
    n_in = shape[0] if transpose else shape[1]
    X = torch.as_tensor(rng.standard_normal((4, n_in)).astype(np.float32)).to(cuda)
    op = lambda v: bpl.cusparse_csr_matvec(data, indices, indptr, v, shape=shape, transpose=transpose)
    torch.testing.assert_close(vmap(op)(X), torch.stack([op(X[b]) for b in range(4)]), rtol=1e-5, atol=1e-4)
    primal, tangent = jvp(op, (X[0],), (X[1],))
    want = (X[1].double() @ dense) if transpose else (dense @ X[1].double())
    torch.testing.assert_close(tangent.double(), want, rtol=1e-5, atol=1e-4)


def test_jitconn_vmap_equals_a_loop_and_jvp_is_the_operator_on_the_tangent(cuda):
  rng = np.random.default_rng(54)
  shape, prob, seed = (100, 200), 0.1, 1234
  ev = torch.as_tensor(rng.random((10, 200)) < 0.3).to(cuda)
  for op in (lambda e: bpl.event_matvec_prob_conn_homo_weight(e, 1.5, conn_prob=prob, shape=shape, seed=seed),
             lambda e: bpl.event_matvec_prob_conn_uniform_weight(e, w_low=-1., w_high=1., conn_prob=prob, shape=shape, seed=seed),
             lambda e: bpl.event_matvec_prob_conn_normal_weight(e, w_mu=0., w_sigma=0.1, conn_prob=prob, shape=shape, seed=seed)):
    assert torch.equal(vmap(op)(ev), torch.stack([op(ev[b]) for b in range(10)]))
  X = torch.as_tensor(rng.standard_normal((6, 200)).astype(np.float32)).to(cuda)
  mv = lambda v: bpl.matvec_prob_conn_normal_weight(v, w_mu=0., w_sigma=0.1, conn_prob=prob, shape=shape, seed=seed)
  assert torch.equal(vmap(mv)(X), torch.stack([mv(X[b]) for b in range(6)]))
  primal, tangent = jvp(mv, (X[0],), (X[1],))
  assert torch.equal(primal, mv(X[0])) and torch.equal(tangent, mv(X[1]))
  evf = ev[0].float()
  emv = lambda e: bpl.event_matvec_prob_conn_normal_weight(e, w_mu=0., w_sigma=0.1, conn_prob=prob, shape=shape, seed=seed)
  _, t2 = jvp(emv, (evf,), (X[2],))
  assert torch.equal(t2, mv(X[2]))           # event_matvec.py:242-260: the dense-vector operator on events_dot


def test_matmat_vmap_over_a_batch_of_matrices(cuda):
  rng = np.random.default_rng(55)
  Xs = torch.as_tensor(rng.standard_normal((3, 8, 100)).astype(np.float32)).to(cuda)
  for version in ('v1', 'v2'):
    op = lambda X: bpl.matmat_prob_conn_normal_weight(X, w_mu=0., w_sigma=0.1, conn_prob=0.1, shape=(100, 60), seed=3,
                                                      version=version)
    assert torch.equal(vmap(op)(Xs), torch.stack([op(Xs[b]) for b in range(3)]))
