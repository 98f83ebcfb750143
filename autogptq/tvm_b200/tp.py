"""Tensor-parallel sharding of packed GPTQ layers.

The reference has no tensor parallelism (its only multi-GPU code places whole decoder layers on
different devices, ``quantization/opt.py:270-304``); these are the slicing rules that the packed
format imposes when one linear is split over ranks:

* column-parallel (shard the output features N): take the same columns of ``qweight``, ``scales``
  and ``bias`` and the matching packed words of ``qzeros`` (fields run along N, so the cut must fall
  on a multiple of 32 columns); ``g_idx`` is shared.  Outputs are concatenated; no exchange.
* row-parallel (shard the input features K): the cut falls on quantisation-group boundaries, so a
  rank takes whole groups: rows ``[g_a*gs, g_b*gs)`` of ``qweight`` (32/bits rows per word),
  rows ``[g_a, g_b)`` of ``scales`` and ``qzeros``, and a local ``g_idx``.  Outputs are summed
  (one all-reduce); the bias is added by rank 0 only.  Needs ``g_idx[k] == k // gs``
  (act-order layers are re-ordered before they are cut).
"""
from __future__ import annotations

from typing import List, Tuple

import torch

from .synth import PackedLayer


def split_sizes(total: int, parts: int, unit: int) -> List[int]:
    """``parts`` multiples of ``unit`` that sum to ``total`` (itself a multiple of ``unit``), as even as possible."""
    if total % unit != 0:
        raise ValueError(f"{total} is not a multiple of {unit}")
    base, extra = divmod(total // unit, parts)
    return [(base + (1 if r < extra else 0)) * unit for r in range(parts)]


def _bounds(sizes: List[int], rank: int) -> Tuple[int, int]:
    a = sum(sizes[:rank])
    return a, a + sizes[rank]


def shard_column(layer: PackedLayer, rank: int, world: int) -> PackedLayer:
    a, b = _bounds(split_sizes(layer.N, world, 32), rank)
    if a == b:
        raise ValueError("more ranks than 32-column blocks")
    wa, wb = a // 32 * layer.bits, b // 32 * layer.bits
    return PackedLayer(layer.bits, layer.group_size, layer.K, b - a,
                       layer.qweight[:, a:b].contiguous(), layer.qzeros[:, wa:wb].contiguous(),
                       layer.scales[:, a:b].contiguous(), layer.g_idx.clone(),
                       None if layer.bias is None else layer.bias[a:b].contiguous())


def shard_row(layer: PackedLayer, rank: int, world: int) -> Tuple[PackedLayer, Tuple[int, int]]:
    """Returns the shard and the range of input features ``[k_a, k_b)`` it consumes."""
    gs = layer.group_size if layer.group_size != -1 else layer.K
    if layer.K % gs != 0:
        raise ValueError("row-parallel sharding needs K to be a multiple of group_size")
    trivial = torch.arange(layer.K, device=layer.g_idx.device) // gs
    if not torch.equal(layer.g_idx.long(), trivial):
        raise ValueError("row-parallel sharding needs g_idx == k // group_size; re-order act-order layers first")
    unit = gs if gs % 32 == 0 else gs * 32   # whole groups and whole packed words
    k_a, k_b = _bounds(split_sizes(layer.K, world, unit), rank)
    if k_a == k_b:
        raise ValueError("more ranks than quantisation groups")
    ra, rb = k_a // 32 * layer.bits, k_b // 32 * layer.bits
    ga, gb = k_a // gs, k_b // gs
    shard = PackedLayer(layer.bits, layer.group_size, k_b - k_a, layer.N,
                        layer.qweight[ra:rb].contiguous(), layer.qzeros[ga:gb].contiguous(),
                        layer.scales[ga:gb].contiguous(),
                        (torch.arange(k_b - k_a, device=layer.g_idx.device) // gs).to(torch.int32),
                        layer.bias if (layer.bias is not None and rank == 0) else None)
    return shard, (k_a, k_b)
