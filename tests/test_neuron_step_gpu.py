"""The fused caller step (conductance decay + LIF update + spike compaction) and the list-driven products against a
float32 numpy restatement and the CPU oracle of the product, over a recurrent excitatory / inhibitory network of the
shape of the reference's example (brainpylib/_src/op_register/tests/ei_net.py:57-72: 3200 + 800 neurons, fixed
connection probability 0.02, g_max 0.6 / 6.7, reversal 0 / -80 mV, tau 5 / 10 ms).  Weights are homogeneous per
projection, so every sum adds equal values and is independent of the order of the additions: membrane potentials,
conductances and spike trains must agree BIT FOR BIT over the whole run."""
import numpy as np
import pytest
import torch

import cases
import brainpylib_b200 as bpl
from brainpylib_b200 import neuron_ops
from oracle import cpu, neuron as oracle_neuron

pytestmark = pytest.mark.gpu


def _network(n_exc, n_inh, prob, seed):
  n = n_exc + n_inh
  rng = np.random.default_rng(seed)
  mats = []
  for lo, hi, w in ((0, n_exc, 0.6), (n_exc, n, 6.7)):       # rows outside the population are empty
    lens = np.zeros(n, dtype=np.int64)
    lens[lo:hi] = rng.binomial(n, prob, hi - lo)
    indptr = np.zeros(n + 1, dtype=np.int32)
    np.cumsum(lens, out=indptr[1:])
    indices = rng.integers(0, n, int(lens.sum()), dtype=np.int32)
    mats.append((np.full(indices.shape[0], w, dtype=np.float32), indices, indptr))
  return n, mats, rng


@pytest.mark.parametrize('n_exc,n_inh,steps', [(3200, 800, 120), (9000, 2100, 40)])
def test_fused_step_network_matches_the_restatement_bit_for_bit(cuda, n_exc, n_inh, steps):
  n, mats, rng = _network(n_exc, n_inh, 0.02, 5)
  p = neuron_ops.LifExpParams(dt=0.1, tau_syn=[5.0, 10.0], E_rev=[0.0, -80.0], ext_input=20.0, V_rest=-60.0, V_th=-50.0,
                              V_reset=-60.0, R=1.0, tau=20.0, tau_ref=5.0)
  V0 = (rng.standard_normal(n) * 2.0 - 55.0).astype(np.float32)
  # CPU
  V_c, g_c, y_c = V0.copy(), np.zeros((2, n), np.float32), np.zeros((2, n), np.float32)
  tl_c = np.full(n, -1e7, dtype=np.float32)
  # GPU
  V_g, g_g, y_g = torch.as_tensor(V0).to(cuda), torch.zeros(2, n, device=cuda), torch.zeros(2, n, device=cuda)
  tl_g = torch.full((n,), -1e7, device=cuda)
  d_mats = [tuple(torch.as_tensor(a).to(cuda) for a in m) for m in mats]
  total_spikes = 0
  for s in range(steps):
    t = np.float32(s * p.dt)
    sp_c = oracle_neuron.lif_exp_step(y_c, g_c, V_c, tl_c, syn_decay=p.syn_decay, E_rev=p.E_rev, ext_input=p.ext_input,
                                      V_rest=p.V_rest, V_th=p.V_th, V_reset=p.V_reset, R=p.R, lif_decay=p.lif_decay,
                                      tau_ref=p.tau_ref, t=t)
    for c, (data, indices, indptr) in enumerate(mats):
      y_c[c] = cpu.event_csr_matvec(data, indices, indptr, sp_c, shape=(n, n), transpose=True)
    sp_g, lst = bpl.lif_exp_step(y_g, g_g, V_g, tl_g, p, float(t))
    for c, (data, indices, indptr) in enumerate(d_mats):
      bpl.event_csr_matvec_from_list(data, indices, indptr, lst, y_g[c], shape=(n, n))
    assert np.array_equal(sp_g.cpu().numpy(), sp_c), f'spikes differ at step {s}'
    total_spikes += int(sp_c.sum())
  assert total_spikes > 50, 'the network never fired: the test would prove nothing'
  assert V_g.cpu().numpy().tobytes() == V_c.tobytes()
  assert g_g.cpu().numpy().tobytes() == g_c.tobytes()
  assert y_g.cpu().numpy().tobytes() == y_c.tobytes()
  assert tl_g.cpu().numpy().tobytes() == tl_c.tobytes()


def test_spike_list_of_the_fused_step_drives_both_storage_formats(cuda):
  """One step on 50,000 neurons with ~2 % above threshold: the list the fused step writes gives the same product as
  the event vector it also returns, on the CSR matrix and on the prepared (column-blocked) matrix."""
  n = 50_000
  rng = np.random.default_rng(9)
  data, indices, indptr, rng = cases.csr_case((n, n), 0.0005, 7)
  t = [torch.as_tensor(a).to(cuda) for a in (data, indices, indptr)]
  p = neuron_ops.LifExpParams(dt=0.1, tau_syn=[5.0], E_rev=[0.0])
  V = torch.as_tensor(np.where(rng.random(n) < 0.02, -40.0, -60.0).astype(np.float32)).to(cuda)
  y, g, tl = torch.zeros(n, device=cuda), torch.zeros(n, device=cuda), torch.full((n,), -1e7, device=cuda)
  spikes, lst = bpl.lif_exp_step(y, g, V, tl, p, 0.0)
  assert 500 < int(spikes.sum()) < 1500 and not y.any()
  want = bpl.event_csr_matvec(*t, spikes, shape=(n, n), transpose=True)
  a = bpl.event_csr_matvec_from_list(*t, lst, torch.zeros(n, device=cuda), shape=(n, n))
  torch.testing.assert_close(a, want, rtol=1e-5, atol=1e-4)
  prepared = bpl.prepare_event_csr(*t, shape=(n, n))
  b = bpl.event_csr_matvec_from_list(None, None, None, lst, torch.zeros(n, device=cuda), shape=(n, n), prepared=prepared)
  torch.testing.assert_close(b, want, rtol=1e-5, atol=1e-4)
  assert torch.equal(V[spikes > 0], torch.full((int(spikes.sum()),), -60.0, device=cuda))     # reset where it fired
