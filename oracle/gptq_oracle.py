"""CPU oracle for the GPTQ QuantLinear forward path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU, the arithmetic of AutoGPTQ's torch
dequantise-then-matmul path, which is the numerical definition that the CUDA
kernels of this repository are checked against.  It is imported only by the
test-suite, by the smoke check and by the benchmark's CPU-baseline leg; the
product never routes through it.

Reference being restated (paths inside LeiWang1999/AutoGPTQ.tvm):

* ``auto_gptq/nn_modules/qlinear.py:197-243`` -- unpack ``qzeros`` / ``qweight``,
  ``W = scales[g_idx] * (q - z[g_idx])`` in fp16, ``out = x.half() @ W``.
* ``auto_gptq/nn_modules/qlinear.py:77-175``  -- ``pack``.

Parity status: PINNED.  ``tests/golden/*.npz`` were produced by running the
reference file itself (loaded by path) on seeded inputs; ``tests/test_oracle.py``
checks every function here bit-for-bit against those vectors, and, when the
reference tree is present, against the live reference as well.

Layout rules (all integers are little-endian bit streams):

* ``qweight`` int32 ``[K/32*bits, N]``: for bits in {2,4,8} word ``r`` of column
  ``n`` holds rows ``k = r*pf + j`` (``pf = 32/bits``) at bit ``bits*j``.  For
  bits == 3 three consecutive words form one 96-bit stream and row
  ``k = 32*t + j`` sits at bits ``[3j, 3j+3)`` of triple ``t``.
* ``qzeros`` int32 ``[G, N/32*bits]``: the same packing along the N axis; the
  stored field is ``zero - 1`` and is NOT masked after the ``+1``.
* ``scales`` fp16 ``[G, N]``; ``g_idx`` int32 ``[K]`` maps a row to its group.
"""
from __future__ import annotations

import math

import numpy as np
import torch

SUPPORTED_BITS = (2, 3, 4, 8)


# --------------------------------------------------------------------------------------
# integer unpacking
# --------------------------------------------------------------------------------------
def _unpack_stream(words: np.ndarray, bits: int) -> np.ndarray:
    """Unpack along axis 0.  ``words`` is uint32 ``[R, C]``; returns uint8/uint16
    ``[R*32/bits, C]`` where output row ``i`` is the ``i``-th ``bits``-wide field of
    the little-endian bit stream formed by each column's words.

    For bits in {2,4,8} this is ``(word >> bits*j) & maxq``
    (qlinear.py:211-215); for bits == 3 it is the 96-bit-per-triple stream that
    qlinear.py:229-236 decodes with its shift table and two straddle fix-ups.
    """
    assert bits in SUPPORTED_BITS
    words = np.ascontiguousarray(words).view(np.uint32) if words.dtype != np.uint32 else words
    R, C = words.shape
    maxq = (1 << bits) - 1
    out_dtype = np.uint16 if bits == 8 else np.uint8
    if bits in (2, 4, 8):
        pf = 32 // bits
        shifts = (np.arange(pf, dtype=np.uint32) * bits)[None, :, None]
        q = (words[:, None, :] >> shifts) & np.uint32(maxq)
        return q.reshape(R * pf, C).astype(out_dtype)
    assert R % 3 == 0, "3-bit packing needs whole triples of words"
    w = words.reshape(R // 3, 3, C).astype(np.uint64)
    lo = w[:, 0] | (w[:, 1] << np.uint64(32))            # stream bits 0..63
    hi = (w[:, 1] >> np.uint64(16)) | (w[:, 2] << np.uint64(16))  # stream bits 48..111
    out = np.empty((R // 3, 32, C), dtype=out_dtype)
    for j in range(32):
        b = 3 * j
        if b + 3 <= 64:
            out[:, j] = ((lo >> np.uint64(b)) & np.uint64(7)).astype(out_dtype)
        else:
            out[:, j] = ((hi >> np.uint64(b - 48)) & np.uint64(7)).astype(out_dtype)
    return out.reshape(R // 3 * 32, C)


def unpack_qweight(qweight, bits: int) -> np.ndarray:
    """``q[k, n]`` as int8 (int16 for 8-bit), shape ``[K, N]`` -- qlinear.py:211-215, 229-236."""
    qw = _as_numpy(qweight).view(np.uint32)
    q = _unpack_stream(qw, bits)
    return q.astype(np.int16 if bits == 8 else np.int8)


def unpack_qzeros(qzeros, bits: int) -> np.ndarray:
    """``z[g, n] = field + 1`` as int8 (int16 for 8-bit), shape ``[G, N]``.

    qlinear.py:201-209 (2/4/8-bit) and :217-227 (3-bit).  The ``+1`` is applied
    after masking and is not masked again: a stored 4-bit field of 15 means
    zero-point 16.
    """
    qz = _as_numpy(qzeros).view(np.uint32)
    z = _unpack_stream(np.ascontiguousarray(qz.T), bits).T  # packing runs along N
    z = z.astype(np.int16 if bits == 8 else np.int8) + 1
    return np.ascontiguousarray(z)


def _as_numpy(t) -> np.ndarray:
    if isinstance(t, torch.Tensor):
        return t.detach().cpu().contiguous().numpy()
    return np.ascontiguousarray(t)


# --------------------------------------------------------------------------------------
# dequantisation and forward
# --------------------------------------------------------------------------------------
def dequantize(qweight, qzeros, scales, g_idx, bits: int):
    """Return ``(q, z, W)``: int8 ``[K,N]``, int8 ``[G,N]`` and fp16 ``[K,N]``.

    ``W[k,n] = scales[g_idx[k], n] * (q[k,n] - z[g_idx[k], n])`` evaluated as in
    qlinear.py:242: the difference is an int8 (exact), it is converted to fp16
    (exact) and multiplied by the fp16 scale with a single rounding.  numpy's
    float16 multiply rounds the exact fp32 product once, which is that result.
    """
    q = unpack_qweight(qweight, bits)
    z = unpack_qzeros(qzeros, bits)
    s = _as_numpy(scales)
    assert s.dtype == np.float16
    g = _as_numpy(g_idx).astype(np.int64)
    diff = (q.astype(np.int16) - z[g].astype(np.int16)).astype(np.float16)
    W = s[g] * diff
    return q, z, W


def forward_fp64(x, W, bias=None) -> np.ndarray:
    """High-precision product of fp16 ``x`` with the fp16 dequantised ``W``: the
    centre of the output tolerance band (fp32-accumulate reference of the contract)."""
    xf = _as_numpy(x).astype(np.float64).reshape(-1, W.shape[0])
    out = xf @ W.astype(np.float64)
    if bias is not None:
        out = out + _as_numpy(bias).astype(np.float64)
    return out


def output_tolerance(x, W) -> np.ndarray:
    """Per-row absolute tolerance ``1e-2 * ||x_row||_2 * max|W|`` of the output contract."""
    xf = _as_numpy(x).astype(np.float64).reshape(-1, W.shape[0])
    return 1e-2 * np.linalg.norm(xf, axis=1, keepdims=True) * float(np.abs(W.astype(np.float64)).max())


class TorchQuantLinearOracle:
    """The reference forward, step for step, on torch CPU tensors.

    Follows qlinear.py:197-247: broadcast-shift unpack of ``qzeros`` and
    ``qweight``, gather of scale / zero rows by ``g_idx``, fp16 dequantisation and
    ``torch.matmul(x.half(), W)``, then ``+ bias``.  This is the routine the
    benchmark times as the CPU baseline (kind "port"), so it deliberately keeps
    the reference's sequence of full-size temporaries.
    """

    def __init__(self, bits, qweight, qzeros, scales, g_idx, bias=None):
        if bits not in SUPPORTED_BITS:
            raise NotImplementedError("Only 2,3,4,8 bits are supported.")
        self.bits = bits
        self.qweight = torch.as_tensor(qweight)
        self.qzeros = torch.as_tensor(qzeros)
        self.scales = torch.as_tensor(scales)
        self.g_idx = torch.as_tensor(g_idx)
        self.bias = None if bias is None else torch.as_tensor(bias)
        self.outfeatures = self.qweight.shape[1]

    def _unpack_along0(self, words: torch.Tensor) -> torch.Tensor:
        bits = self.bits
        if bits in (2, 4, 8):
            pf = 32 // bits
            sh = torch.arange(0, 32, bits, dtype=torch.int32).reshape(1, pf, 1)
            q = torch.bitwise_right_shift(words.unsqueeze(1).expand(-1, pf, -1), sh)
            q = q.to(torch.int16 if bits == 8 else torch.int8)
            q = torch.bitwise_and(q, (1 << bits) - 1)
            return q.reshape(-1, words.shape[1])
        t = words.reshape(words.shape[0] // 3, 3, words.shape[1]).to(torch.int64) & 0xFFFFFFFF
        lo = t[:, 0] | (t[:, 1] << 32)
        hi = (t[:, 1] >> 16) | (t[:, 2] << 16)
        sh_lo = torch.arange(0, 63, 3, dtype=torch.int64).reshape(1, 21, 1)       # j = 0..20
        sh_hi = torch.arange(63 - 48, 96 - 48, 3, dtype=torch.int64).reshape(1, 11, 1)  # j = 21..31
        a = (lo.unsqueeze(1) >> sh_lo) & 7
        b = (hi.unsqueeze(1) >> sh_hi) & 7
        return torch.cat([a, b], dim=1).to(torch.int8).reshape(-1, words.shape[1])

    def dequantize(self):
        z = self._unpack_along0(self.qzeros.t().contiguous()).t() + 1
        q = self._unpack_along0(self.qweight)
        g = self.g_idx.long()
        return self.scales[g] * (q - z[g])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out_shape = x.shape[:-1] + (self.outfeatures,)
        x = x.reshape(-1, x.shape[-1])
        out = torch.matmul(x.half(), self.dequantize())
        out = out.reshape(out_shape)
        return out + self.bias if self.bias is not None else out


# --------------------------------------------------------------------------------------
# packing
# --------------------------------------------------------------------------------------
def _pack_stream(vals: np.ndarray, bits: int) -> np.ndarray:
    """Inverse of :func:`_unpack_stream`: ``vals`` uint32 ``[R, C]`` -> uint32 words
    ``[R*bits/32, C]``.  Values wider than ``bits`` bleed into the neighbouring
    fields exactly as the reference's un-masked ``|=`` does (qlinear.py:111-134)."""
    vals = vals.astype(np.uint32)
    R, C = vals.shape
    assert R % 32 == 0
    if bits in (2, 4, 8):
        pf = 32 // bits
        v = vals.reshape(R // pf, pf, C)
        out = np.zeros((R // pf, C), dtype=np.uint32)
        for j in range(pf):
            out |= v[:, j] << np.uint32(bits * j)
        return out
    v = vals.reshape(R // 32, 32, C)
    out = np.zeros((R // 32, 3, C), dtype=np.uint32)
    for j in range(10):
        out[:, 0] |= v[:, j] << np.uint32(3 * j)
    out[:, 0] |= v[:, 10] << np.uint32(30)
    out[:, 1] |= (v[:, 10] >> np.uint32(2)) & np.uint32(1)
    for j in range(11, 21):
        out[:, 1] |= v[:, j] << np.uint32(3 * (j - 11) + 1)
    out[:, 1] |= v[:, 21] << np.uint32(31)
    out[:, 2] |= (v[:, 21] >> np.uint32(1)) & np.uint32(3)
    for j in range(22, 32):
        out[:, 2] |= v[:, j] << np.uint32(3 * (j - 22) + 2)
    return out.reshape(R // 32 * 3, C)


def pack(weight, scales, zeros, g_idx, bits: int):
    """Restatement of ``QuantLinear.pack`` (qlinear.py:77-175).

    ``weight`` fp ``[N, K]`` (``nn.Linear`` layout), ``scales`` / ``zeros`` fp
    ``[N, G]``, ``g_idx`` int ``[K]``.  Returns ``(qweight, qzeros, scales_fp16)``
    as int32 ``[K/32*bits, N]``, int32 ``[G, N/32*bits]`` and fp16 ``[G, N]``.

    ``intweight[k] = round((W[:,k] + (zero*scale)[g]) / fp16(scale)[g])`` uses
    round-half-to-even in fp32, with the fp32 ``zero*scale`` product in the
    numerator and the fp16-rounded scale in the denominator, as the reference does.
    """
    W = torch.as_tensor(weight).float()
    scales_t = torch.as_tensor(scales).float().t().contiguous()
    zeros_t = torch.as_tensor(zeros).float().t().contiguous()
    g = torch.as_tensor(g_idx).long()
    scale_zeros = zeros_t * scales_t
    scales_h = scales_t.clone().half()
    intweight = torch.round((W.t() + scale_zeros[g]) / scales_h[g]).to(torch.int)
    qweight = _pack_stream(intweight.numpy().astype(np.uint32), bits).astype(np.int32)
    z = (zeros_t - 1).numpy().astype(np.uint32)
    qzeros = _pack_stream(np.ascontiguousarray(z.T), bits).T.astype(np.int32)
    return qweight, np.ascontiguousarray(qzeros), scales_h.numpy()


def expected_shapes(bits: int, K: int, N: int, group_size: int):
    gs = group_size if group_size != -1 else K
    G = math.ceil(K / gs)
    return (K // 32 * bits, N), (G, N // 32 * bits), (G, N)
