"""B200-native (sm_100a) backend for the GPTQ ``QuantLinear`` forward path.

Drop-in for the TVM backend of LeiWang1999/AutoGPTQ.tvm
(``auto_gptq/nn_modules/qlinear_tvm.py``): the same ``QuantLinear(bits, groupsize,
infeatures, outfeatures, bias)`` module surface on the standard AutoGPTQ packed
buffers, evaluated by hand-written CUDA kernels behind a C ABI.

Sub-modules load on first use: ``synth`` (synthetic layers) needs only torch, while ``QuantLinear`` and ``ops``
bind ``libb200gptq.so`` -- and fail loudly when it is missing, there is no fallback.
"""
import importlib

__all__ = ["QuantLinear", "ops"]

_SUBMODULES = {"ops", "synth", "qlinear", "tp", "decoder", "modeling", "exchange", "build", "_lib"}


def __getattr__(name):
    if name == "QuantLinear":
        return importlib.import_module(".qlinear", __name__).QuantLinear
    if name in _SUBMODULES:
        return importlib.import_module("." + name, __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
