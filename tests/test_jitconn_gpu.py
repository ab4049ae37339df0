"""GPU parity of the just-in-time-connectivity operators.

Bitwise oracle: the reference's own CUDA kernels (lib/gpu_jitconn_*.cu compiled for sm_100a
into oracle/_ref/libref_gpu.so) on the same inputs and descriptors.  Row-parallel outputs
must be bit-identical (same streams, same per-row summation order); column-parallel outputs
are sums of atomics and are compared with rtol 1e-5 / atol 1e-5 * expected in-degree, except
homogeneous event products, which are integer counts and exact.

Second check: the CPU oracle (oracle/jitconn_oracle.cu), which calls the same cuRAND header on
the host.  Its `logf` is glibc's, so a sampled position may differ where the quotient sits
within one ulp of an integer; the oracle counts such draws ("fragile") and the comparison
allows that many rows to differ.
"""
import numpy as np
import pytest
import torch

import cases
import brainpylib_b200 as bpl
from brainpylib_b200 import gpu_ops, jitconn_ops
from oracle import cpu, ref

pytestmark = pytest.mark.gpu
needs_ref_gpu = pytest.mark.skipif(not ref.available_gpu(), reason='oracle/_ref/libref_gpu.so not built')

KINDS = [('homo', 0., 0.), ('uniform', -0.1, 0.2), ('normal', 0., 0.01)]
ORACLE_KIND = {'homo': cpu.W_HOMO, 'uniform': cpu.W_UNIFORM, 'normal': cpu.W_NORMAL}


def descriptor(kind, n_row, n_col, seed, conn_prob, w1, w2):
  return jitconn_ops._descriptor(kind, n_row, n_col, seed, conn_prob, w1, w2)


def call_event(events, kind, w1, w2, conn_prob, shape, seed, transpose, odp):
  if kind == 'homo':
    return bpl.event_matvec_prob_conn_homo_weight(events, 1., conn_prob=conn_prob, shape=shape, seed=seed,
                                                  transpose=transpose, outdim_parallel=odp)
  if kind == 'uniform':
    return bpl.event_matvec_prob_conn_uniform_weight(events, w_low=w1, w_high=w1 + w2, conn_prob=conn_prob,
                                                     shape=shape, seed=seed, transpose=transpose, outdim_parallel=odp)
  return bpl.event_matvec_prob_conn_normal_weight(events, w_mu=w1, w_sigma=w2, conn_prob=conn_prob, shape=shape,
                                                  seed=seed, transpose=transpose, outdim_parallel=odp)


def call_dense(vector, kind, w1, w2, conn_prob, shape, seed, transpose, odp):
  if kind == 'homo':
    return bpl.matvec_prob_conn_homo_weight(vector, 1., conn_prob=conn_prob, shape=shape, seed=seed,
                                            transpose=transpose, outdim_parallel=odp)
  if kind == 'uniform':
    return bpl.matvec_prob_conn_uniform_weight(vector, w_low=w1, w_high=w1 + w2, conn_prob=conn_prob, shape=shape,
                                               seed=seed, transpose=transpose, outdim_parallel=odp)
  return bpl.matvec_prob_conn_normal_weight(vector, w_mu=w1, w_sigma=w2, conn_prob=conn_prob, shape=shape,
                                            seed=seed, transpose=transpose, outdim_parallel=odp)


@needs_ref_gpu
@pytest.mark.parametrize('kind,w1,w2', KINDS)
@pytest.mark.parametrize('odp', [True, False])
@pytest.mark.parametrize('ev_dtype', [torch.bool, torch.float32, torch.float64])
def test_event_matvec_equals_reference_kernels(cuda, kind, w1, w2, odp, ev_dtype):
  g = torch.Generator(device='cpu').manual_seed(5)
  for shape, prob in [((100, 200), 0.1), ((10, 1000), 0.01), ((1000, 10), 0.4), ((2, 1000), 0.1), ((1000, 2), 0.5),
                      ((5000, 6000), 0.02)]:
    for transpose in (False, True):
      n_in = shape[0] if transpose else shape[1]
      n_out = shape[1] if transpose else shape[0]
      ev = torch.rand(n_in, generator=g) < 0.2
      if ev_dtype != torch.bool:
        ev = ev.to(ev_dtype) * (torch.rand(n_in, generator=g).to(ev_dtype) + 0.5)   # values other than 1
      ev = ev.to(cuda)
      y = call_event(ev, kind, w1, w2, prob, shape, 1234, transpose, odp)
      y_ref = torch.full_like(y, float('nan'))
      tname = 'float' if y.dtype == torch.float32 else 'double'
      ename = 'bool' if ev_dtype == torch.bool else tname
      name = f'gpu_event_matvec{"" if odp else "_atomic"}_prob_{kind}_v2_{tname}_{ename}'
      ref.gpu_call(name, [ev, y_ref], descriptor(kind, n_out, n_in, 1234, prob, w1, w2))
      if odp or kind == 'homo':
        assert torch.equal(y, y_ref), (shape, transpose, (y - y_ref).abs().max())
      else:
        torch.testing.assert_close(y, y_ref, rtol=1e-5, atol=1e-5 * max(1., prob * n_in))


@needs_ref_gpu
@pytest.mark.parametrize('kind,w1,w2', KINDS)
@pytest.mark.parametrize('odp', [True, False])
@pytest.mark.parametrize('dtype', [torch.float32, torch.float64])
def test_matvec_equals_reference_kernels(cuda, kind, w1, w2, odp, dtype):
  g = torch.Generator(device='cpu').manual_seed(6)
  for shape, prob in [((100, 200), 0.1), ((10, 1000), 0.01), ((1000, 10), 0.4), ((3000, 2500), 0.05)]:
    for transpose in (False, True):
      n_in = shape[0] if transpose else shape[1]
      n_out = shape[1] if transpose else shape[0]
      v = torch.randn(n_in, generator=g, dtype=dtype).to(cuda)
      y = call_dense(v, kind, w1, w2, prob, shape, 99, transpose, odp)
      y_ref = torch.full_like(y, float('nan'))
      tname = 'float' if dtype == torch.float32 else 'double'
      name = f'gpu_matvec{"" if odp else "_atomic"}_prob_{kind}_v2_{tname}'
      ref.gpu_call(name, [v, y_ref], descriptor(kind, n_out, n_in, 99, prob, w1, w2))
      if odp:
        assert torch.equal(y, y_ref), (shape, transpose, (y - y_ref).abs().max())
      else:
        torch.testing.assert_close(y, y_ref, rtol=1e-5 if dtype == torch.float32 else 1e-12,
                                   atol=1e-5 * max(1., prob * n_in) * (1. if kind == 'homo' else 0.2))


@needs_ref_gpu
@pytest.mark.parametrize('kind,w1,w2', KINDS)
@pytest.mark.parametrize('dtype', [torch.float32, torch.float64])
def test_matvec_v1_equals_reference_kernels(cuda, kind, w1, w2, dtype):
  """version='v1': a Bernoulli test per (row, column) with the raw probability in the descriptor
  (lib/gpu_jitconn_matvec.cu:10-54,141-187,284-331)."""
  g = torch.Generator(device='cpu').manual_seed(14)
  for shape, prob in [((100, 200), 0.1), ((10, 1000), 0.01), ((1000, 10), 0.4), ((300, 777), 0.5), ((2, 1000), 1.0)]:
    for transpose in (False, True):
      n_in = shape[0] if transpose else shape[1]
      n_out = shape[1] if transpose else shape[0]
      v = torch.randn(n_in, generator=g, dtype=dtype).to(cuda)
      if kind == 'homo':
        y = bpl.matvec_prob_conn_homo_weight(v, 1., conn_prob=prob, shape=shape, seed=5, transpose=transpose,
                                             version='v1')
        opaque = gpu_ops.build_jitconn_prob_homo_descriptor(n_out, n_in, 5, prob)
      elif kind == 'uniform':
        y = bpl.matvec_prob_conn_uniform_weight(v, w_low=w1, w_high=w1 + w2, conn_prob=prob, shape=shape, seed=5,
                                                transpose=transpose, version='v1')
        opaque = gpu_ops.build_jitconn_prob_uniform_descriptor(n_out, n_in, 5, prob, w1, w2)
      else:
        y = bpl.matvec_prob_conn_normal_weight(v, w_mu=w1, w_sigma=w2, conn_prob=prob, shape=shape, seed=5,
                                               transpose=transpose, version='v1')
        opaque = gpu_ops.build_jitconn_prob_normal_descriptor(n_out, n_in, 5, prob, w1, w2)
      y_ref = torch.full_like(y, float('nan'))
      tname = 'float' if dtype == torch.float32 else 'double'
      ref.gpu_call(f'gpu_matvec_prob_{kind}_v1_{tname}', [v, y_ref], opaque)
      assert torch.equal(y, y_ref), (shape, transpose, (y - y_ref).abs().max())
  with pytest.raises(bpl.GPUOperatorNotFound):
    bpl.matvec_prob_conn_homo_weight(torch.zeros(10, device=cuda), 1., conn_prob=0.1, shape=(5, 10), seed=1,
                                     outdim_parallel=False, version='v1')


@needs_ref_gpu
def test_mask_kernel_path_equals_reference(cuda):
  """Large enough for the shared-memory bitmask kernel (>= 4096 rows), bool and float events."""
  shape, prob = (20000, 30000), 0.01
  g = torch.Generator(device='cpu').manual_seed(7)
  ev = (torch.rand(shape[1], generator=g) < 0.05).to(cuda)
  for kind, w1, w2 in KINDS:
    for e in (ev, ev.float() * 2.5):
      y = call_event(e, kind, w1, w2, prob, shape, 42, False, True)
      y_ref = torch.empty_like(y)
      ename = 'bool' if e.dtype == torch.bool else 'float'
      ref.gpu_call(f'gpu_event_matvec_prob_{kind}_v2_float_{ename}', [e, y_ref],
                   descriptor(kind, shape[0], shape[1], 42, prob, w1, w2))
      assert torch.equal(y, y_ref), kind


@pytest.mark.parametrize('kind,w1,w2', KINDS)
def test_against_cpu_oracle(cuda, kind, w1, w2):
  shape, prob, seed = (2000, 3000), 0.05, 4321
  rng = np.random.default_rng(8)
  ev = rng.random(shape[1]) < 0.1
  y = call_event(torch.as_tensor(ev).to(cuda), kind, w1, w2, prob, shape, seed, False, True).cpu().numpy()
  want, info = cpu.jitconn_event_matvec(ev, kind=ORACLE_KIND[kind], w1=w1, w2=w2, conn_prob=prob, shape=shape,
                                        seed=seed, return_info=True)
  assert 0.8 < info['connections'] / (prob * shape[0] * shape[1]) < 1.2
  tol = dict(rtol=1e-5, atol=1e-6) if kind != 'normal' else dict(rtol=1e-4, atol=1e-5)   # host sinf/cosf vs device
  bad = ~np.isclose(y, want, **tol)
  assert bad.sum() <= info['fragile'], (bad.sum(), info)
  # dense vector, both orientations
  x = rng.standard_normal(shape[1]).astype(np.float32)
  for odp in (True, False):
    y = call_dense(torch.as_tensor(x).to(cuda), kind, w1, w2, prob, shape, seed, False, odp).cpu().numpy()
    want, info = cpu.jitconn_matvec(x, kind=ORACLE_KIND[kind], w1=w1, w2=w2, conn_prob=prob, shape=shape, seed=seed,
                                    outdim_parallel=odp, return_info=True)
    bad = ~np.isclose(y, want, rtol=1e-4, atol=1e-3 if kind == 'homo' else 1e-4)
    assert bad.sum() <= 4 * info['fragile'] + (0 if odp else 0), (odp, bad.sum(), info)


def test_relations_of_the_reference_tests(cuda):
  """brainpylib/_src/jitconn_ops/tests/test_event_matvec.py:63-87 and test_matvec.py:55-81."""
  g = torch.Generator(device='cpu').manual_seed(9)
  for shape in cases.JITCONN_SHAPES:
    for prob in (0.01, 0.1, 0.5):
      for kind, w1, w2 in KINDS:
        for transpose in (False, True):
          for odp in (True, False):
            n_in = shape[0] if transpose else shape[1]
            ev = (torch.rand(n_in, generator=g) < 0.1).to(cuda)
            r1 = call_event(ev, kind, w1, w2, prob, shape, 1234, transpose, odp)
            r2 = call_event(ev, kind, w1, w2, prob, shape, 1234, transpose, odp)
            if odp or kind == 'homo':
              assert torch.equal(r1, r2)
            else:
              torch.testing.assert_close(r1, r2, rtol=1e-5, atol=1e-6)
            r3 = call_event(ev, kind, w1, w2, prob, shape[::-1], 1234, not transpose, odp)
            torch.testing.assert_close(r1, r3, rtol=1e-5, atol=1e-6)
            # bool events == float 0/1 events
            r4 = call_event(ev.float(), kind, w1, w2, prob, shape, 1234, transpose, odp)
            torch.testing.assert_close(r1, r4, rtol=1e-5, atol=1e-6)
            # dense product on the 0/1 vector
            r5 = call_dense(ev.float(), kind, w1, w2, prob, shape, 1234, transpose, odp)
            torch.testing.assert_close(r1, r5, rtol=1e-5, atol=1e-6)


def test_row_and_column_parallel_are_transposes(cuda):
  """(shape, T, odp) and (shape, not T, not odp) walk the same streams: <M x, z> == <x, M^T z>, and
  the autograd rule (brainpylib/_src/jitconn_ops/matvec.py:393-402) relies on it."""
  shape, prob, seed = (700, 900), 0.05, 77
  g = torch.Generator(device='cpu').manual_seed(10)
  for kind, w1, w2 in KINDS:
    x = torch.randn(shape[1], generator=g, dtype=torch.float64).to(cuda)
    z = torch.randn(shape[0], generator=g, dtype=torch.float64).to(cuda)
    mx = call_dense(x, kind, w1, w2, prob, shape, seed, False, True)
    mtz = call_dense(z, kind, w1, w2, prob, shape, seed, True, False)
    torch.testing.assert_close(torch.dot(mx, z), torch.dot(x, mtz), rtol=1e-9, atol=1e-9)
    xg = x.clone().requires_grad_(True)
    y = call_dense(xg, kind, w1, w2, prob, shape, seed, False, True)
    gx, = torch.autograd.grad(y, xg, z)
    torch.testing.assert_close(gx, mtz, rtol=1e-12, atol=1e-12)
    eg = (torch.rand(shape[1], generator=g) < 0.3).double().to(cuda).requires_grad_(True)
    ye = call_event(eg, kind, w1, w2, prob, shape, seed, False, True)
    ge, = torch.autograd.grad(ye, eg, z)
    torch.testing.assert_close(ge, mtz, rtol=1e-12, atol=1e-12)


def test_edge_parameters(cuda):
  """conn_prob 1e-4, 0.5 and 1.0; a single input; seeds next to 2^32 (seed + row wraps)."""
  ev = torch.ones(300, dtype=torch.bool, device=cuda)
  y = bpl.event_matvec_prob_conn_homo_weight(ev, 1., conn_prob=1.0, shape=(50, 300), seed=3)
  # every gap is 1 when conn_prob >= 1: positions 1..299 connect, position 0 does not
  assert torch.equal(y, torch.full((50,), 299., device=cuda))
  y = bpl.event_matvec_prob_conn_homo_weight(ev, 1., conn_prob=1e-4, shape=(50, 300), seed=3)
  assert y.sum().item() <= 50
  y1 = bpl.event_matvec_prob_conn_homo_weight(ev[:1], 1., conn_prob=0.5, shape=(50, 1), seed=3)
  assert y1.shape == (50,) and y1.max().item() <= 1
  for seed in (2 ** 32 - 3, 2 ** 32 - 1):
    a = bpl.event_matvec_prob_conn_homo_weight(ev, 1., conn_prob=0.1, shape=(50, 300), seed=seed)
    want = cpu.jitconn_event_matvec(np.ones(300, np.bool_), kind=cpu.W_HOMO, conn_prob=0.1, shape=(50, 300), seed=seed)
    assert (a.cpu().numpy() != want).sum() <= 1
    # rows 3.. of the wrapped seed are rows 0.. of seed 0
    if seed == 2 ** 32 - 3:
      b = bpl.event_matvec_prob_conn_homo_weight(ev, 1., conn_prob=0.1, shape=(47, 300), seed=0)
      assert torch.equal(a[3:], b)


@needs_ref_gpu
@pytest.mark.parametrize('kind,w1,w2', KINDS[1:])
@pytest.mark.parametrize('dtype', [torch.float32, torch.float64])
def test_matmat_equals_reference_kernels(cuda, kind, w1, w2, dtype):
  g = torch.Generator(device='cpu').manual_seed(11)
  # The reference's uniform wrapper sizes its grid as m * n / SIZE threads (lib/gpu_jitconn_matmat.cu:386-398),
  # which leaves columns uncomputed unless m is a multiple of its row-group SIZE (8, 16, 24 or 32):
  # it is only comparable for such m.  The normal wrapper rounds up (:302-314) and takes any m.
  for m in ((8, 16, 64) if kind == 'uniform' else (5, 8, 15, 33, 64)):
    for shape, prob in [((100, 200), 0.1), ((10, 1000), 0.05), ((1000, 10), 0.2), ((200, 200), 0.01),
                        ((1500, 700), 0.02)]:
      # The reference evaluates X[(m_i + i) * k + pos] for row groups that are not full and for the padding
      # threads of its last block, whose m_i = thread / n * SIZE can lie far beyond m when n is small
      # (lib/gpu_jitconn_matmat.cu:248,265): give it a zero-padded copy large enough for every such read.
      X = torch.randn(m, shape[0], generator=g, dtype=dtype).to(cuda)
      pad_rows = ((m + 31) // 32 + 256 // shape[1] + 3) * 32
      pad = torch.zeros(pad_rows * shape[0], dtype=dtype, device=cuda)
      pad[: m * shape[0]] = X.reshape(-1)
      if kind == 'uniform':
        Y = bpl.matmat_prob_conn_uniform_weight(X, w_low=w1, w_high=w1 + w2, conn_prob=prob, shape=shape, seed=7)
      else:
        Y = bpl.matmat_prob_conn_normal_weight(X, w_mu=w1, w_sigma=w2, conn_prob=prob, shape=shape, seed=7)
      Y_ref = torch.empty_like(Y)
      tname = 'float' if dtype == torch.float32 else 'double'
      opaque = gpu_ops.build_matmat_jit_prob_descriptor1(m, shape[0], shape[1], 7, jitconn_ops._log_p(prob), w1, w2)
      ref.gpu_call(f'gpu_matmat_prob_prob_{kind}_{tname}_v1', [pad, Y_ref], opaque)
      assert torch.equal(Y, Y_ref), (m, shape, (Y - Y_ref).abs().max())


def test_matmat_equals_matvec_per_row(cuda):
  """brainpylib/_src/jitconn_ops/tests/matmat_testcase.py:59-78,119-138."""
  g = torch.Generator(device='cpu').manual_seed(12)
  for m in (5, 33):
    for shape in cases.MATMAT_SHAPES:
      for prob in (0.01, 0.2):
        X = torch.randn(m, shape[0], generator=g).to(cuda)
        Y = bpl.matmat_prob_conn_normal_weight(X, w_mu=0., w_sigma=0.01, conn_prob=prob, shape=shape, seed=1234)
        Y2 = bpl.matmat_prob_conn_normal_weight(X, w_mu=0., w_sigma=0.01, conn_prob=prob, shape=shape, seed=1234)
        assert torch.equal(Y, Y2)
        rows = torch.stack([bpl.matvec_prob_conn_normal_weight(X[r], w_mu=0., w_sigma=0.01, conn_prob=prob,
                                                               shape=shape, seed=1234, transpose=True)
                            for r in range(m)])
        assert torch.equal(Y, rows)
        U = bpl.matmat_prob_conn_uniform_weight(X, w_low=-0.1, w_high=0.1, conn_prob=prob, shape=shape, seed=1234)
        rows = torch.stack([bpl.matvec_prob_conn_uniform_weight(X[r], w_low=-0.1, w_high=0.1, conn_prob=prob,
                                                                shape=shape, seed=1234, transpose=True)
                            for r in range(m)])
        assert torch.equal(U, rows)


def test_matmat_against_cpu_oracle(cuda):
  rng = np.random.default_rng(13)
  X = rng.standard_normal((16, 3000)).astype(np.float32)
  Y = bpl.matmat_prob_conn_uniform_weight(torch.as_tensor(X).to(cuda), w_low=-0.1, w_high=0.1, conn_prob=0.02,
                                          shape=(3000, 500), seed=7).cpu().numpy()
  want, info = cpu.jitconn_matmat(X, kind=cpu.W_UNIFORM, w1=-0.1, w2=0.2, conn_prob=0.02, shape=(3000, 500), seed=7,
                                  return_info=True)
  bad_cols = (~np.isclose(Y, want, rtol=1e-5, atol=1e-6)).any(axis=0)
  assert bad_cols.sum() <= info['fragile'], (bad_cols.sum(), info)


@pytest.mark.parametrize('kind', ['uniform', 'normal'])
@pytest.mark.parametrize('world', [2, 3, 8])
def test_matmat_column_shards_concatenate_to_the_full_product(cuda, kind, world):
  """Sharding by output column needs no exchange: every column has its own stream (seed + column), so the
  ranks' outputs side by side are bit-identical to the single-device result."""
  from brainpylib_b200 import sharded
  m, k, n = 40, 300, 1000 + world   # ragged last shard
  X = torch.randn(m, k, device=cuda)
  kw = dict(kind=kind, w1=0.1, w2=0.5, conn_prob=0.05, shape=(k, n), seed=4294967290)   # seed + column wraps
  full = jitconn_ops.matmat_raw(X, **kw)
  parts = [sharded.matmat_column_shard(X, rank=r, world=world, **kw) for r in range(world)]
  assert sum(p.shape[1] for p in parts) == n
  assert torch.equal(torch.cat(parts, dim=1), full)


# ------------------------------------------------------------------------------------------
# matmat versions 'v2' and 'v3': other random matrices than 'v1', each bit for bit against its own reference
# kernel (lib/gpu_jitconn_matmat.cu:138-231 and :19-135).
# ------------------------------------------------------------------------------------------
@pytest.mark.skipif(not ref.available_gpu(), reason='oracle/_ref/libref_gpu.so not built')
@pytest.mark.parametrize('dtype', [torch.float32, torch.float64])
@pytest.mark.parametrize('m', [5, 8, 16, 24, 32, 40, 64])
def test_matmat_v2_equals_reference_kernel(cuda, m, dtype):
  """The reference reads X beyond its m rows when m is not a multiple of its row group (and in padding warps):
  it gets a zero-padded copy large enough for every such read; only the store is guarded there."""
  tname = 'float' if dtype == torch.float32 else 'double'
  for shape, prob in (((100, 200), 0.1), ((1000, 7), 0.02), ((33, 257), 0.3)):
    X = torch.randn(m, shape[0], dtype=dtype, device=cuda, generator=torch.Generator(device=cuda).manual_seed(m))
    Y = bpl.matmat_prob_conn_normal_weight(X, w_mu=0.1, w_sigma=0.02, conn_prob=prob, shape=shape, seed=11, version='v2')
    pad = torch.zeros((m + 64 + 16 * 32) * shape[0], dtype=dtype, device=cuda)
    pad[: m * shape[0]] = X.reshape(-1)
    Y_ref = torch.full((m, shape[1]), float('nan'), dtype=dtype, device=cuda)
    opaque = gpu_ops.build_matmat_jit_prob_descriptor1(m, shape[0], shape[1], 11, jitconn_ops._log_p(prob), 0.1, 0.02)
    ref.gpu_call(f'gpu_matmat_prob_prob_normal_{tname}_v2', [pad, Y_ref], opaque)
    assert torch.equal(Y, Y_ref), (m, shape, (Y - Y_ref).abs().max().item())
    assert not torch.equal(Y, bpl.matmat_prob_conn_normal_weight(X, w_mu=0.1, w_sigma=0.02, conn_prob=prob, shape=shape,
                                                                 seed=11))   # another matrix than v1's


@pytest.mark.skipif(not ref.available_gpu(), reason='oracle/_ref/libref_gpu.so not built')
@pytest.mark.parametrize('dtype', [torch.float32, torch.float64])
def test_matmat_v3_equals_reference_kernel_where_the_reference_is_defined(cuda, dtype):
  """m = 32 only: one warp per block.  For other m the reference either never terminates (rows beyond m never see
  the position advance, lib/gpu_jitconn_matmat.cu:40-55) or races on its shared arrays (no barrier between a
  round's reads and the next round's writes), so it is not run there."""
  tname = 'float' if dtype == torch.float32 else 'double'
  m = 32
  for shape, prob in (((100, 200), 0.1), ((1000, 7), 0.02), ((33, 257), 0.3)):
    X = torch.randn(m, shape[0], dtype=dtype, device=cuda, generator=torch.Generator(device=cuda).manual_seed(3))
    Y = bpl.matmat_prob_conn_normal_weight(X, w_mu=0.1, w_sigma=0.02, conn_prob=prob, shape=shape, seed=11, version='v3')
    Y_ref = torch.full((m, shape[1]), float('nan'), dtype=dtype, device=cuda)
    opaque = gpu_ops.build_matmat_jit_prob_descriptor1(m, shape[0], shape[1], 11, jitconn_ops._log_p(prob), 0.1, 0.02)
    ref.gpu_call(f'gpu_matmat_prob_prob_normal_{tname}_v3', [X, Y_ref], opaque)
    assert torch.equal(Y, Y_ref), (shape, (Y - Y_ref).abs().max().item())


def test_matmat_v3_and_v2_relations_where_the_reference_cannot_run(cuda):
  """Any m: deterministic; v3's rows of one block share one connectivity, so scaling X scales Y exactly (power of
  two) and a row of zeros gives zeros; v2 is linear in X in the same sense."""
  for version in ('v2', 'v3'):
    for m in (5, 33, 70, 600):
      shape, prob = (300, 50), 0.05
      X = torch.randn(m, shape[0], device=cuda, generator=torch.Generator(device=cuda).manual_seed(m))
      kw = dict(w_mu=0., w_sigma=0.5, conn_prob=prob, shape=shape, seed=5, version=version)
      Y = bpl.matmat_prob_conn_normal_weight(X, **kw)
      assert Y.shape == (m, shape[1]) and torch.isfinite(Y).all() and Y.abs().sum() > 0
      assert torch.equal(Y, bpl.matmat_prob_conn_normal_weight(X, **kw))
      assert torch.equal(bpl.matmat_prob_conn_normal_weight(4 * X, **kw), 4 * Y)
      X0 = X.clone()
      X0[m // 2] = 0
      assert not bpl.matmat_prob_conn_normal_weight(X0, **kw)[m // 2].any()


# ------------------------------------------------------------------------------------------
# The counter-based ("v1") event products: gpu_event_matvec_prob_{homo,uniform,normal}_{float,double}.  The
# reference's wrappers for these targets cannot run (host dereference of the device-side event count), so the pin
# is the CPU restatement of the kernel text (oracle.cpu.jitconn_event_matvec_v1): integer-exact generators, so
# homogeneous and uniform results must agree bit for bit; normal weights go through log / sqrt / cos in double on
# both sides and are compared at 1e-6 relative.
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize('dtype', [torch.float32, torch.float64])
@pytest.mark.parametrize('kind,w1,w2', [('homo', 0., 0.), ('uniform', -0.1, 0.2), ('normal', 0.05, 0.01)])
@pytest.mark.parametrize('shape,prob,rate', [((100, 200), 0.1, 0.2), ((1000, 10), 0.4, 0.5), ((3, 3000), 0.02, 0.3),
                                             ((700, 900), 0.05, 0.0), ((513, 300), 0.5, 1.0)])
def test_counter_based_event_matvec_matches_the_kernel_text(cuda, shape, prob, rate, kind, w1, w2, dtype):
  rng = np.random.default_rng(17)
  seed = 2_654_435_761                      # a large seed: the one-step generators mix small seeds poorly
  ev = rng.random(shape[1]) < rate
  ids = np.flatnonzero(ev).astype(np.int32)
  np_dtype = np.float32 if dtype == torch.float32 else np.float64
  want = cpu.jitconn_event_matvec_v1(ids, ids.shape[0], kind=['homo', 'uniform', 'normal'].index(kind), w1=w1, w2=w2,
                                     conn_prob=prob, n_row=shape[0], n_col=shape[1], seed=seed, dtype=np_dtype)
  events = torch.as_tensor(ev).to(cuda) if dtype == torch.float32 else torch.as_tensor(ev.astype(np.float64)).to(cuda)
  ops = {'homo': lambda e, **kw: bpl.event_matvec_prob_conn_homo_weight(e, 1.0, **kw),
         'uniform': lambda e, **kw: bpl.event_matvec_prob_conn_uniform_weight(e, w_low=w1, w_high=w1 + w2, **kw),
         'normal': lambda e, **kw: bpl.event_matvec_prob_conn_normal_weight(e, w_mu=w1, w_sigma=w2, **kw)}
  y = ops[kind](events, conn_prob=prob, shape=shape, seed=seed, version='v1')
  assert y.dtype == dtype and y.shape == (shape[0],)
  y = y.cpu().numpy()
  if kind == 'normal':
    np.testing.assert_allclose(y, want, rtol=1e-6, atol=1e-6)
  else:
    assert y.tobytes() == want.tobytes(), np.abs(y - want).max()
  # (the density of the generated matrix is NOT asserted: one step of lfsr113 from a raw seed mixes poorly, e.g. 6 %
  #  instead of 40 % for 10 input columns; that is the generator the reference's kernel text defines)
  # transpose only swaps which side is the output: (shape, T) == (shape[::-1], not T), as for v2
  if rate > 0 and kind != 'normal':
    ev_t = rng.random(shape[0]) < rate
    e_t = torch.as_tensor(ev_t).to(cuda) if dtype == torch.float32 else torch.as_tensor(ev_t.astype(np.float64)).to(cuda)
    a = ops[kind](e_t, conn_prob=prob, shape=shape, seed=seed, version='v1', transpose=True)
    b = ops[kind](e_t, conn_prob=prob, shape=shape[::-1], seed=seed, version='v1', transpose=False)
    assert torch.equal(a, b)


def test_counter_based_event_matvec_refuses_what_it_has_no_kernel_for(cuda):
  ev = torch.ones(10, dtype=torch.bool, device=cuda)
  with pytest.raises(ValueError):
    bpl.event_matvec_prob_conn_homo_weight(ev, 1.0, conn_prob=0.1, shape=(5, 10), seed=1, version='v1', outdim_parallel=False)
  with pytest.raises(ValueError):
    bpl.event_matvec_prob_conn_homo_weight(ev, 1.0, conn_prob=0.1, shape=(5, 10), seed=1, version='v3')


@pytest.mark.parametrize('kind,w1,w2', KINDS[1:])
@pytest.mark.parametrize('dtype', [torch.float32, torch.float64])
def test_matmat_from_lists_is_bit_identical_to_the_inline_kernel(cuda, kind, w1, w2, dtype):
  """The *_v1_ws targets (streams generated once into lists, then multiplied) against the *_v1 targets (the
  reference's structure: stream regenerated per 32 rows) over ragged sizes; then with a list capacity of 3 slots,
  where most columns overflow and are recomputed by the inline kernel; then with a byte budget that walks the
  columns in several chunks; then both."""
  import ctypes
  from brainpylib_b200 import _lib
  lib = _lib.lib()
  lib.bpl_matmat_list_limits_for_tests.argtypes = [ctypes.c_uint32, ctypes.c_size_t]
  lib.bpl_matmat_list_limits_for_tests.restype = None
  g = torch.Generator(device='cpu').manual_seed(17)
  sizes = [(5, (100, 200), 0.1), (33, (1000, 10), 0.2), (64, (777, 1301), 0.03), (40, (3000, 2500), 0.01),
           (1, (64, 513), 1.0)]
  try:
    for cap, budget in ((0, 0), (3, 0), (0, 40000), (7, 40000)):
      lib.bpl_matmat_list_limits_for_tests(cap, budget)
      for m, shape, prob in sizes:
        X = torch.randn(m, shape[0], generator=g, dtype=dtype).to(cuda)
        kw = dict(kind=kind, w1=w1, w2=w2, conn_prob=prob, shape=shape, seed=2 ** 32 - 100)   # the seed wraps
        plain = jitconn_ops.matmat_raw(X, workspace=False, **kw)
        listed = jitconn_ops.matmat_raw(X, **kw)
        assert torch.equal(plain, listed), (cap, budget, m, shape, prob)
  finally:
    lib.bpl_matmat_list_limits_for_tests(0, 0)
