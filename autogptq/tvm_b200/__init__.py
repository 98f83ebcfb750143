"""B200-native (sm_100a) backend for the GPTQ ``QuantLinear`` forward path.

Drop-in for the TVM backend of LeiWang1999/AutoGPTQ.tvm
(``auto_gptq/nn_modules/qlinear_tvm.py``): the same ``QuantLinear(bits, groupsize,
infeatures, outfeatures, bias)`` module surface on the standard AutoGPTQ packed
buffers, evaluated by hand-written CUDA kernels behind a C ABI.
"""
from .qlinear import QuantLinear  # noqa: F401
from . import ops  # noqa: F401

__all__ = ["QuantLinear", "ops"]
