"""brainpylib_b200: synaptic propagation on NVIDIA B200 behind brainpylib's operator API.

The operator modules keep the names of the reference package (``event_ops``,
``sparse_ops``, ``jitconn_ops``, ``compat``, ``gpu_ops``); arrays are torch CUDA tensors.
Every operator runs a hand-written sm_100a kernel of ``libbrainpylib_b200.so``; without
that library an operator raises :class:`GPUOperatorNotFound` (there is no CPU fallback).
"""
__version__ = '0.1.0'

from .errors import GPUOperatorNotFound
from . import gpu_ops
from . import event_ops
from .event_ops import *
from . import sparse_ops
from .sparse_ops import *
from . import jitconn_ops
from .jitconn_ops import *
from . import compat
from .compat import *
from . import neuron_ops
from .neuron_ops import *
from . import host_steps
from .host_steps import HostSteps
