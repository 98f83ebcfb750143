"""Seeded synthetic GPTQ layers with the value distributions of the benchmark configs.

Real checkpoints are not available offline, so the benchmark and the tests draw
packed buffers directly: every int32 bit pattern is a valid packing of uniform
integer fields, zero-point fields are uniform as well (stored ``zero - 1``), scales
are ``|N(0, 0.02)| + 1e-3`` in fp16, and ``g_idx`` is either ``k // group_size`` or
a random permutation of the rows cut into groups (act-order).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class PackedLayer:
    bits: int
    group_size: int
    K: int
    N: int
    qweight: torch.Tensor
    qzeros: torch.Tensor
    scales: torch.Tensor
    g_idx: torch.Tensor
    bias: Optional[torch.Tensor] = None

    def to(self, device):
        mv = lambda t: None if t is None else t.to(device)
        return PackedLayer(self.bits, self.group_size, self.K, self.N, mv(self.qweight), mv(self.qzeros),
                           mv(self.scales), mv(self.g_idx), mv(self.bias))

    def weight_bytes(self) -> int:
        return self.qweight.numel() * 4

    def algorithmic_bytes(self, M: int = 1) -> int:
        """qweight + qzeros + scales + g_idx + x + y, the bytes one forward must move."""
        return (self.qweight.numel() * 4 + self.qzeros.numel() * 4 + self.scales.numel() * 2 +
                self.g_idx.numel() * 4 + M * self.K * 2 + M * self.N * 2)


def _randint32(shape, gen, device):
    return torch.randint(-2**31, 2**31 - 1, shape, generator=gen, dtype=torch.int64, device=device).to(torch.int32)


def make_layer(bits: int, K: int, N: int, group_size: int = 128, act_order: bool = False, bias: bool = False,
               seed: int = 0, device="cpu", scale_mult: float = 1.0) -> PackedLayer:
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(seed)
    gs = group_size if group_size != -1 else K
    G = math.ceil(K / gs)
    qweight = _randint32((K // 32 * bits, N), gen, device)
    qzeros = _randint32((G, N // 32 * bits), gen, device)
    scales = ((torch.randn((G, N), generator=gen, device=device).abs() * 0.02 + 1e-3) * scale_mult).half()
    if act_order:
        g_idx = (torch.randperm(K, generator=gen, device=device) // gs).to(torch.int32)
    else:
        g_idx = (torch.arange(K, device=device) // gs).to(torch.int32)
    b = (torch.randn(N, generator=gen, device=device) * 0.1).half() if bias else None
    return PackedLayer(bits, group_size, K, N, qweight, qzeros, scales, g_idx, b)


def make_x(M: int, K: int, seed: int = 0, device="cpu") -> torch.Tensor:
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(seed + 7919)
    return torch.randn((M, K), generator=gen, device=device).half()


# The benchmark configurations (shapes of BASELINE.json's `configs`).
CONFIGS = {
    "c0_gemv_b4_k4096_n4096": dict(bits=4, K=4096, N=4096, group_size=128, act_order=False, M=[1]),
    "c1_gemv_b3_k4096_n11008_act": dict(bits=3, K=4096, N=11008, group_size=128, act_order=True, M=[1]),
    "c2_gemm_b4_k4096_n12288": dict(bits=4, K=4096, N=12288, group_size=128, act_order=False,
                                    M=[16, 128, 512, 2048]),
}
