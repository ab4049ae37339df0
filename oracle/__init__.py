"""CPU checkers for the synaptic-propagation path.  TEST INFRASTRUCTURE ONLY.

``oracle.cpu``  numpy-facing wrappers of ``liboracle.so`` (this repository's CPU
                restatement of the reference algorithms).
``oracle.ref``  ctypes access to the reference's own kernels compiled into
                ``oracle/_ref/`` (CPU always; CUDA when a GPU is present).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU legs of ``bench.py`` may
import this package; the product (``brainpylib_b200``) never does.
"""
