"""``torch.library`` registration of the QuantLinear product, so that it can be traced.

``QuantLinear.forward`` calls the C ABI through ctypes, which ``torch.compile`` / ``torch.export`` cannot look into.
``torch.ops.b200gptq.quant_matmul`` is the same product as one opaque operator with a shape rule: a traced module
records one node per layer and runs the library's kernels at run time.  ``QuantLinear.forward`` goes through it
whenever it is being compiled and keeps its prepared per-layer plans otherwise.

The dispatch is the stateless form of the reference's per-M kernel choice
(auto_gptq/nn_modules/tvm_untils/pycuda_warpper.py:138-189): up to 8 rows the decode GEMV, otherwise the tcgen05
GEMM when the layer's group layout allows it, otherwise GEMV passes (up to 64 rows) or one dequantisation and a dense
product.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

GEMV_MAX_M = 8


@torch.library.custom_op("b200gptq::quant_matmul", mutates_args=(), device_types="cuda")
def quant_matmul(x: Tensor, qweight: Tensor, qzeros: Tensor, scales: Tensor, g_idx: Optional[Tensor],
                 x_perm: Optional[Tensor], bias: Optional[Tensor], bits: int, group_size: int,
                 gemm_ok: bool) -> Tensor:
    """``x`` fp16 ``[M, K]`` (contiguous) times the packed layer -> fp16 ``[M, N]``.  ``g_idx`` / ``x_perm`` are the
    run-time layout of the layer (``None`` for groups ``k // group_size`` / no gather), ``gemm_ok`` says that every
    aligned 32-row block lies in one group (what the tensor-core kernel needs)."""
    from . import ops
    M = x.shape[0]
    N = qweight.shape[1]
    args = (qweight, qzeros, scales, g_idx, bits, group_size)
    kw = dict(bias=bias, x_perm=x_perm)
    with torch.cuda.device(x.device):
        if M <= GEMV_MAX_M:
            return ops.gemv(x, *args, **kw)
        if gemm_ok:
            return ops.gemm(x, *args, **kw)
        if M > 64:
            _, W = ops.dequantize(qweight, qzeros, scales, g_idx, bits, group_size, want_q=False)
            xg = x if x_perm is None else x.index_select(1, x_perm.long())
            y = xg @ W
            return y if bias is None else y + bias
        y = torch.empty((M, N), dtype=torch.float16, device=x.device)
        for m0 in range(0, M, GEMV_MAX_M):
            ops.gemv(x[m0:m0 + GEMV_MAX_M], *args, out=y[m0:m0 + GEMV_MAX_M], **kw)
        return y


@quant_matmul.register_fake
def _(x, qweight, qzeros, scales, g_idx, x_perm, bias, bits, group_size, gemm_ok):
    torch._check(x.dim() == 2, lambda: "x must be [M, K]")
    torch._check(x.shape[1] * bits == qweight.shape[0] * 32, lambda: "x and qweight disagree about K")
    return x.new_empty((x.shape[0], qweight.shape[1]), dtype=torch.float16)


__all__ = ["quant_matmul"]
