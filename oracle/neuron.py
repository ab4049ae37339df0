"""float32 array restatement of the fused neuron / synapse step (brainpylib_b200/csrc/neuron_kernels.cu).
TEST INFRASTRUCTURE ONLY.

The formulas are BrainPy's exponential synapse and ``LIF`` neuron with exponential-Euler integration, as used by the
reference's network example brainpylib/_src/op_register/tests/ei_net.py:47-72 (BrainPy is a dependency outside the
reference tree, so its published update rule is restated; parity with BrainPy itself is unpinned).  numpy rounds every
float32 product and sum on its own, which is exactly what the kernel does with its unfused arithmetic."""
import numpy as np


def lif_exp_step(y, g, V, t_last, *, syn_decay, E_rev, ext_input, V_rest, V_th, V_reset, R, lif_decay, tau_ref, t):
  """In-place on g, V, t_last (float32); y (K, n) is consumed and cleared.  Returns the spikes (float32 0/1)."""
  f = np.float32
  k = g.shape[0]
  inp = np.full(V.shape, f(ext_input), dtype=np.float32)
  for c in range(k):
    g[c] = g[c] * f(syn_decay[c]) + y[c]
    y[c] = 0
    inp = inp + g[c] * (f(E_rev[c]) - V)
  refractory = (f(t) - t_last) <= f(tau_ref)
  v_inf = f(V_rest) + f(R) * inp
  v_new = v_inf + (V - v_inf) * f(lif_decay)
  v_new = np.where(refractory, V, v_new).astype(np.float32)
  spike = v_new >= f(V_th)
  t_last[spike] = f(t)
  V[:] = np.where(spike, f(V_reset), v_new)
  return spike.astype(np.float32)
