"""``QuantLinear`` -- the module that ``make_quant(..., use_tvm=True)`` installs.

Mirrors the constructor / ``pack`` / ``forward`` surface of the reference's TVM
module (``auto_gptq/nn_modules/qlinear_tvm.py:10-158``) but keeps the standard
AutoGPTQ buffers of ``auto_gptq/nn_modules/qlinear.py:40-59`` (``qweight``,
``qzeros``, ``scales``, ``g_idx``, ``bias``), so ordinary GPTQ checkpoints load
unchanged.  ``forward`` runs on the GPU only: M <= 8 rows go to the decode GEMV,
more rows to the tcgen05 dequant-GEMM.  There is no M padding, no per-shape
kernel cache and no tuner (the reference's ``tvm_untils/cache.py`` and
``pycuda_warpper.py`` have no counterpart here).
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn as nn

from . import ops

GEMV_MAX_M = 8


def _pack_fields(vals: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack ``vals`` (int64 ``[R, C]``, R % 32 == 0) along dim 0 into int32 words.

    2/4/8 bits: field j of a word at bit ``bits*j``.  3 bits: 32 fields form a
    96-bit little-endian stream over three words.  Over-wide values spill into
    the neighbouring fields exactly like the reference's un-masked ``|=``
    (qlinear.py:111-134).
    """
    R, C = vals.shape
    if bits in (2, 4, 8):
        pf = 32 // bits
        v = vals.reshape(R // pf, pf, C)
        shifts = (torch.arange(pf, dtype=torch.int64) * bits).reshape(1, pf, 1)
        words = torch.zeros((R // pf, C), dtype=torch.int64)
        for j in range(pf):
            words |= (v[:, j] << (bits * j)) & 0xFFFFFFFF
        del shifts
    else:
        v = vals.reshape(R // 32, 32, C)
        words = torch.zeros((R // 32, 3, C), dtype=torch.int64)
        for j in range(32):
            bit = 3 * j
            wi, sh = bit // 32, bit % 32
            words[:, wi] |= (v[:, j] << sh) & 0xFFFFFFFF
            if sh > 29:  # the field straddles into the next word
                mask = (1 << (sh + 3 - 32)) - 1
                words[:, wi + 1] |= (v[:, j] >> (32 - sh)) & mask
        words = words.reshape(R // 32 * 3, C)
    words = torch.where(words >= 2**31, words - 2**32, words)
    return words.to(torch.int32)


class QuantLinear(nn.Module):
    def __init__(self, bits, groupsize, infeatures, outfeatures, bias):
        super().__init__()
        if bits not in [2, 3, 4, 8]:
            raise NotImplementedError("Only 2,3,4,8 bits are supported.")
        if infeatures % 32 != 0 or outfeatures % 32 != 0:
            raise ValueError("infeatures and outfeatures must be multiples of 32 (the packed format needs it)")
        self.infeatures = infeatures
        self.outfeatures = outfeatures
        self.bits = bits
        self.groupsize = groupsize if groupsize != -1 else infeatures
        self.maxq = 2 ** self.bits - 1
        G = math.ceil(infeatures / self.groupsize)
        self.register_buffer("qweight", torch.zeros((infeatures // 32 * bits, outfeatures), dtype=torch.int32))
        self.register_buffer("qzeros", torch.zeros((G, outfeatures // 32 * bits), dtype=torch.int32))
        self.register_buffer("scales", torch.zeros((G, outfeatures), dtype=torch.float16))
        self.register_buffer("g_idx", (torch.arange(infeatures, dtype=torch.int64) // self.groupsize).to(torch.int32))
        if bias:
            self.register_buffer("bias", torch.zeros((outfeatures,), dtype=torch.float16))
        else:
            self.bias = None
        # derived, non-persistent state built by post_init() on the device
        self._ready_for = None
        self._qweight_run = None   # the weights the kernels read: qweight itself or its row-sorted copy
        self._g_idx_run = None     # None => rows use group k // groupsize
        self._x_perm = None        # None => no gather of x
        self._gemm_ok = False      # the run-time layout meets the tensor-core kernel's one-group-per-32-rows rule
        # Row-parallel shard of a tensor-parallel model: forward_reduce() returns the sum over ranks.  `exchange` is an
        # exchange.PeerExchange (fused all-reduce for up to 8 rows), `tp_bias` the full bias that every rank adds after
        # the sum.
        self.exchange = None
        self.tp_bias = None
        # (slices_per_sm, ctas_per_sm) of b200gptq_gemv_tuned, or None for the library defaults
        self.gemv_tuning = None
        self._plans = {}           # row count -> ops.GemvPlan (prepared launches of the decode GEMV)

    # ---- offline packing (CPU) ----------------------------------------------------------
    def pack(self, linear, scales, zeros, g_idx=None):
        """Same contract as ``QuantLinear.pack`` of the reference (qlinear.py:77-175):
        ``scales`` / ``zeros`` are ``[outfeatures, G]``; the integer weight is
        ``round((W + zero*scale) / fp16(scale))`` per row group and ``zeros - 1`` is stored.
        With the layer and the statistics on a CUDA device the whole procedure runs there (the
        reference packs with a Python loop over the rows on the CPU); the result is bit-identical."""
        W = linear.weight.data.clone()
        if isinstance(linear, nn.Conv2d):
            W = W.flatten(1)
        elif type(linear).__name__ == "Conv1D":  # transformers.pytorch_utils.Conv1D keeps [in, out]
            W = W.t()
        self.g_idx = g_idx.clone() if g_idx is not None else self.g_idx
        g = self.g_idx.long()
        scales = scales.t().contiguous()
        zeros = zeros.t().contiguous()
        scale_zeros = zeros * scales
        self.scales = scales.clone().half()
        if linear.bias is not None:
            self.bias = linear.bias.detach().clone().half()
        intweight = torch.round((W.t() + scale_zeros[g]) / self.scales[g]).to(torch.int)
        if W.is_cuda:
            # everything on the GPU: the same element-wise arithmetic, words built by b200gptq_pack_fields
            self.qweight = ops.pack_fields(intweight.contiguous(), self.bits)
            zq = (zeros - 1).to(torch.int64).to(torch.int32)
            self.qzeros = ops.pack_fields(zq.t().contiguous(), self.bits).t().contiguous()
            self._ready_for = None
            return
        intweight = torch.from_numpy(intweight.numpy().astype(np.uint32).astype(np.int64))
        self.qweight = _pack_fields(intweight, self.bits)
        zq = torch.from_numpy((zeros - 1).numpy().astype(np.uint32).astype(np.int64))
        self.qzeros = _pack_fields(zq.t().contiguous(), self.bits).t().contiguous()
        self._ready_for = None

    # ---- device-side preparation ----------------------------------------------------------
    def post_init(self):
        """Build the run-time view of the layer on its current device.

        A layer whose ``g_idx`` is constant over every aligned block of 32 rows is
        used as stored.  Any other ``g_idx`` (act-order checkpoints) is re-ordered
        once so that rows of a group are adjacent; ``forward`` then gathers ``x``
        through the permutation inside the kernels.
        """
        dev = self.qweight.device
        if dev.type != "cuda":
            raise RuntimeError("QuantLinear.post_init needs the module on a CUDA device")
        K = self.infeatures
        g = self.g_idx
        trivial = torch.equal(g, (torch.arange(K, device=dev, dtype=torch.int64) // self.groupsize).to(torch.int32))
        blocks = g.view(K // 32, 32)
        block_uniform = bool((blocks == blocks[:, :1]).all().item())
        if trivial:
            self._qweight_run, self._g_idx_run, self._x_perm = self.qweight, None, None
        elif block_uniform:
            self._qweight_run, self._g_idx_run, self._x_perm = self.qweight, g.contiguous(), None
        else:
            qs, perm, gs = ops.sort_rows(self.qweight.contiguous(), g.contiguous(), self.bits)
            sorted_trivial = torch.equal(
                gs, (torch.arange(K, device=dev, dtype=torch.int64) // self.groupsize).to(torch.int32))
            self._qweight_run, self._x_perm = qs, perm
            self._g_idx_run = None if sorted_trivial else gs
        # the tensor-core kernel takes one group per aligned 32-row block: true for every run-time g_idx built above
        # (block-uniform or sorted by group with whole blocks) except a NULL g_idx with a group size that is no
        # multiple of 32, and a sorted layout whose groups do not fill whole blocks
        g_run = self._g_idx_run
        if g_run is None:
            self._gemm_ok = self.bits in (3, 4) and self.groupsize % 32 == 0
        else:
            b = g_run.view(K // 32, 32)
            self._gemm_ok = self.bits in (3, 4) and bool((b == b[:, :1]).all().item())
        self._plans = {}
        self._ready_for = (self.qweight.data_ptr(), self.g_idx.data_ptr())

    def _ready(self) -> bool:
        b = self._buffers    # (a tensor on another device has another address, so the addresses say it all)
        return self._ready_for == (b["qweight"].data_ptr(), b["g_idx"].data_ptr())

    # ---- forward --------------------------------------------------------------------------
    def forward(self, x):
        if torch.compiler.is_compiling():
            # Traced: one opaque, shape-inferable operator per layer (torch_ops.py).  The run-time layout must exist
            # already (post_init(), which from_quantized and the first eager call run); the prepared plans below are
            # for eager calls.
            from .torch_ops import quant_matmul
            x2 = x.half().reshape(-1, self.infeatures).contiguous()
            y = quant_matmul(x2, self._qweight_run, self.qzeros, self.scales, self._g_idx_run, self._x_perm,
                             self.bias, self.bits, self.groupsize, self._gemm_ok)
            return y.reshape(x.shape[:-1] + (self.outfeatures,))
        if not x.is_cuda:
            raise RuntimeError("QuantLinear.forward needs CUDA tensors: this backend has no CPU path")
        if not self._ready():
            self.post_init()
        # decode: up to 8 rows, already fp16 and contiguous, a plan at hand -- one allocation and one library call
        if x.dtype is torch.float16 and x.is_contiguous() and x.shape[-1] == self.infeatures:
            M = x.numel() // self.infeatures
            if 0 < M <= GEMV_MAX_M:
                plan = self._plans.get((M, self.gemv_tuning))
                if (plan is not None and plan._keep[5] is self._buffers.get("bias", self.__dict__.get("bias"))
                        and x.get_device() == plan._index):
                    return plan.launch(x, x.shape[:-1] + (self.outfeatures,))
        out_shape = x.shape[:-1] + (self.outfeatures,)
        x2 = x.half().reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M = x2.shape[0]
        kw = dict(bias=self.bias, x_perm=self._x_perm)
        args = (self._qweight_run, self.qzeros, self.scales, self._g_idx_run, self.bits, self.groupsize)
        if M <= GEMV_MAX_M:
            key = (M, self.gemv_tuning)
            plan = self._plans.get(key)
            if plan is None or plan._keep[5] is not self.bias:
                plan = self._plans[key] = ops.GemvPlan(self._qweight_run, self.qzeros, self.scales, self._g_idx_run,
                                                     self._x_perm, self.bias, M, self.bits, self.groupsize,
                                                     self.gemv_tuning)
            with torch.cuda.device(x2.device):
                y = plan.run(x2)
        elif self._gemm_ok:
            # measured on B200: from 9 rows on, one tensor-core pass (35-45 us for a 4096 x 12288 layer) beats two
            # or more GEMV passes
            y = ops.gemm(x2, *args, **kw)
        elif M > 64:
            # no tensor-core kernel for this layout and many rows: dequantise once with the library's kernel (the
            # reference's own dequantise-then-matmul order, qlinear.py:242-243) and let the dense product run on the
            # GPU's GEMM library; M / 8 GEMV passes would read the weights M / 8 times
            _, W = ops.dequantize(self._qweight_run, self.qzeros, self.scales, self._g_idx_run, self.bits,
                                  self.groupsize, want_q=False)
            xg = x2 if self._x_perm is None else x2.index_select(1, self._x_perm.long())
            y = xg @ W
            if self.bias is not None:
                y = y + self.bias
        else:
            # 2- and 8-bit layers, and layers whose groups cut through 32-row blocks, have no tensor-core kernel:
            # GEMV passes of up to 8 rows
            y = torch.empty((M, self.outfeatures), dtype=torch.float16, device=x2.device)
            for m0 in range(0, M, GEMV_MAX_M):
                ops.gemv(x2[m0:m0 + GEMV_MAX_M], *args, out=y[m0:m0 + GEMV_MAX_M], **kw)
        return y.reshape(out_shape)

    # ---- the element-wise kernel in front of this layer folded into its read of x (decode batches only) ----
    def can_fold(self, rows: int, input_act: int) -> bool:
        """Whether :meth:`forward_act` / ``forward_reduce(..., input_act)`` can take the activation for ``rows`` rows."""
        if not self._ready():
            self.post_init()
        return rows <= GEMV_MAX_M and ops.can_fold_act(rows, self.infeatures, self.outfeatures, self.bits, self.groupsize,
                                                       self._g_idx_run is not None, self._x_perm is not None, input_act)

    def forward_act(self, u, input_act: int):
        """``forward(act(u))`` in one launch for up to 8 rows: ``input_act = _lib.ACT_SWIGLU`` (``u`` is
        ``[..., 2 * in] = [gate | up]``) or ``_lib.ACT_RELU`` (``b200gptq_gemv_plan_create_ex``).  The caller checks
        :meth:`can_fold` first."""
        if not self._ready():
            self.post_init()
        u2 = u.half().reshape(-1, u.shape[-1])
        if not u2.is_contiguous():
            u2 = u2.contiguous()
        M = u2.shape[0]
        key = (M, self.gemv_tuning, input_act)
        plan = self._plans.get(key)
        if plan is None or plan._keep[5] is not self.bias:
            plan = self._plans[key] = ops.GemvPlan(self._qweight_run, self.qzeros, self.scales, self._g_idx_run,
                                                 self._x_perm, self.bias, M, self.bits, self.groupsize,
                                                 self.gemv_tuning, input_act)
        with torch.cuda.device(u2.device):
            y = plan.run(u2)
        return y.reshape(u.shape[:-1] + (self.outfeatures,))

    def forward_reduce(self, x, input_act: int = 0):
        """Row-parallel forward: this rank's slice of the input in, the complete output (summed over ranks) out.
        Up to 8 rows go through ``b200gptq_gemv_tp`` (sum fused into the kernel, peer memory); more rows use the
        process group's all-reduce."""
        if self.exchange is None:
            raise RuntimeError("forward_reduce needs an exchange (see exchange.PeerExchange)")
        if not self._ready():
            self.post_init()
        x2 = x.half().reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if x2.shape[0] <= GEMV_MAX_M:
            y = ops.gemv_tp(x2, self._qweight_run, self.qzeros, self.scales, self._g_idx_run, self.bits, self.groupsize,
                            self.exchange, bias=self.tp_bias, x_perm=self._x_perm, tuning=self.gemv_tuning,
                            input_act=input_act)
        else:
            if input_act:
                raise ValueError("an input activation is folded for up to 8 rows only")
            import torch.distributed as dist
            saved, self.bias = self.bias, None
            try:
                y = self.forward(x2)
            finally:
                self.bias = saved
            dist.all_reduce(y, group=self.exchange.group)
            if self.tp_bias is not None:
                y = y + self.tp_bias
        return y.reshape(x.shape[:-1] + (self.outfeatures,))

    def extra_repr(self):
        return (f"in={self.infeatures}, out={self.outfeatures}, bits={self.bits}, "
                f"groupsize={self.groupsize}, bias={self.bias is not None}")


__all__ = ["QuantLinear"]
