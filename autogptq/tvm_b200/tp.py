"""Tensor-parallel sharding of packed GPTQ layers.

The reference has no tensor parallelism (its only multi-GPU code places whole decoder layers on
different devices, ``quantization/opt.py:270-304``); these are the slicing rules that the packed
format imposes when one linear is split over ranks:

* column-parallel (shard the output features N): take the same columns of ``qweight``, ``scales``
  and ``bias`` and the matching packed words of ``qzeros`` (fields run along N, so every cut must fall
  on a multiple of 32 columns); ``g_idx`` is shared.  Outputs are concatenated; no exchange.  A fused
  layer (q|k|v, gate|up) is cut part by part, so that a rank owns the same heads / the same slice of
  the FFN width in every part.
* row-parallel (shard the input features K): a rank takes rows ``[k_a, k_b)`` of ``qweight`` (cuts on
  multiples of 32 rows: 32 rows are ``bits`` whole words).  Outputs are summed (one all-reduce); the bias
  is added by rank 0 only.  Two cases:

  - ``g_idx[k] == k // group_size`` and both cuts on group boundaries: the shard is an ordinary layer of
    its own -- rows ``[k_a/gs, k_b/gs)`` of ``scales`` / ``qzeros`` and a local ``g_idx``.
  - anything else (act-order checkpoints, cuts through groups): the shard keeps the GLOBAL group ids of
    its rows and the whole ``scales`` / ``qzeros``: every K shard of an act-order layer touches every
    group (``W[k, n] = scales[g_idx[k], n] * (q[k, n] - zeros[g_idx[k], n])``, reference
    ``auto_gptq/nn_modules/qlinear.py:242``).  Such a shard has few rows per group, so it runs on the
    general GEMV kernel, not the streaming one.

* an act-order layer whose input is an element-wise function of a column-parallel layer's output
  (fc1 -> fc2, gate|up -> down) avoids that: :func:`fold_act_order` re-orders its rows by group once and applies
  the same permutation to the producer's output columns, after which the consumer is an ordinary layer
  (``g_idx == k // group_size``) that is cut on group boundaries, streams, and needs no gather of its input.
  The function computed by the pair does not change.  (o_proj / out_proj cannot use it: their input is laid out by
  attention head.)
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .synth import PackedLayer


def split_sizes(total: int, parts: int, unit: int) -> List[int]:
    """``parts`` multiples of ``unit`` that sum to ``total`` (itself a multiple of ``unit``), as even as possible."""
    if total % unit != 0:
        raise ValueError(f"{total} is not a multiple of {unit}")
    base, extra = divmod(total // unit, parts)
    return [(base + (1 if r < extra else 0)) * unit for r in range(parts)]


def bounds(sizes: Sequence[int], rank: int) -> Tuple[int, int]:
    a = sum(sizes[:rank])
    return a, a + sizes[rank]


def _group_size(layer: PackedLayer) -> int:
    return layer.group_size if layer.group_size != -1 else layer.K


def is_trivial(layer: PackedLayer) -> bool:
    """``g_idx[k] == k // group_size``."""
    gs = _group_size(layer)
    return bool(torch.equal(layer.g_idx.long(), torch.arange(layer.K, device=layer.g_idx.device) // gs))


def take_columns(layer: PackedLayer, ranges: Sequence[Tuple[int, int]]) -> PackedLayer:
    """The layer restricted to the output columns ``[a, b)`` of every range, concatenated in order."""
    cols, words = [], []
    for a, b in ranges:
        if a % 32 or b % 32 or not 0 <= a < b <= layer.N:
            raise ValueError(f"column range [{a}, {b}) must be non-empty, inside the layer and cut on multiples of 32")
        cols.append(torch.arange(a, b, device=layer.qweight.device))
        words.append(torch.arange(a // 32 * layer.bits, b // 32 * layer.bits, device=layer.qweight.device))
    c, w = torch.cat(cols), torch.cat(words)
    return PackedLayer(layer.bits, layer.group_size, layer.K, int(c.numel()),
                       layer.qweight.index_select(1, c).contiguous(), layer.qzeros.index_select(1, w).contiguous(),
                       layer.scales.index_select(1, c).contiguous(), layer.g_idx.clone(),
                       None if layer.bias is None else layer.bias.index_select(0, c).contiguous())


def take_rows(layer: PackedLayer, k_a: int, k_b: int, keep_bias: bool) -> PackedLayer:
    """The layer restricted to the input rows ``[k_a, k_b)`` (see the module docstring for the two cases)."""
    if k_a % 32 or k_b % 32 or not 0 <= k_a < k_b <= layer.K:
        raise ValueError(f"row range [{k_a}, {k_b}) must be non-empty, inside the layer and cut on multiples of 32")
    gs = _group_size(layer)
    ra, rb = k_a // 32 * layer.bits, k_b // 32 * layer.bits
    bias = layer.bias if keep_bias else None
    if is_trivial(layer) and k_a % gs == 0 and (k_b % gs == 0 or k_b == layer.K):
        ga, gb = k_a // gs, -(-k_b // gs)
        return PackedLayer(layer.bits, layer.group_size if layer.group_size != -1 else gs, k_b - k_a, layer.N,
                           layer.qweight[ra:rb].contiguous(), layer.qzeros[ga:gb].contiguous(),
                           layer.scales[ga:gb].contiguous(),
                           (torch.arange(k_b - k_a, device=layer.g_idx.device) // gs).to(torch.int32), bias)
    # global group ids, whole scales / qzeros
    return PackedLayer(layer.bits, layer.group_size if layer.group_size != -1 else gs, k_b - k_a, layer.N,
                       layer.qweight[ra:rb].contiguous(), layer.qzeros.contiguous(), layer.scales.contiguous(),
                       layer.g_idx[k_a:k_b].contiguous(), bias)


def unpack_fields(words: torch.Tensor, bits: int) -> torch.Tensor:
    """Inverse of the packing along dim 0: int32 words ``[R/32*bits, C]`` -> fields int32 ``[R, C]``."""
    w = words.to(torch.int64) & 0xFFFFFFFF
    if bits in (2, 4, 8):
        pf = 32 // bits
        shifts = (torch.arange(pf, device=words.device, dtype=torch.int64) * bits).view(1, pf, 1)
        f = (w.unsqueeze(1) >> shifts) & ((1 << bits) - 1)
        return f.reshape(-1, words.shape[1]).to(torch.int32)
    t = w.reshape(-1, 3, words.shape[1])
    stream_lo = t[:, 0] | (t[:, 1] << 32)            # bits 0..63 of the 96-bit stream
    out = []
    for j in range(32):
        bit = 3 * j
        if bit + 3 <= 64:
            out.append((stream_lo >> bit) & 7)
        else:
            hi = t[:, 2]
            if bit >= 64:
                out.append((hi >> (bit - 64)) & 7)
            else:                                     # field 21 straddles bits 63..65
                out.append(((stream_lo >> bit) & ((1 << (64 - bit)) - 1)) | ((hi & ((1 << (bit + 3 - 64)) - 1)) << (64 - bit)))
    return torch.stack(out, dim=1).reshape(-1, words.shape[1]).to(torch.int32)


def pack_fields_torch(vals: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack int fields ``[R, C]`` (R % 32 == 0, values < 2**bits) along dim 0 into int32 words, on any device."""
    R, C = vals.shape
    v = vals.to(torch.int64)
    if bits in (2, 4, 8):
        pf = 32 // bits
        v = v.reshape(R // pf, pf, C)
        words = torch.zeros((R // pf, C), dtype=torch.int64, device=vals.device)
        for j in range(pf):
            words |= v[:, j] << (bits * j)
    else:
        v = v.reshape(R // 32, 32, C)
        words = torch.zeros((R // 32, 3, C), dtype=torch.int64, device=vals.device)
        for j in range(32):
            bit = 3 * j
            wi, sh = bit // 32, bit % 32
            words[:, wi] |= (v[:, j] << sh) & 0xFFFFFFFF
            if sh > 29:
                words[:, wi + 1] |= v[:, j] >> (32 - sh)
        words = words.reshape(R // 32 * 3, C)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    return words.to(torch.int32)


def permute_columns(layer: PackedLayer, perm: torch.Tensor, parts: int = 1) -> PackedLayer:
    """The layer with its output columns re-ordered inside each of its ``parts`` equal blocks: new column ``j`` of a
    block is old column ``perm[j]`` of that block.  ``qzeros`` is packed along the columns, so its fields are
    unpacked, moved and packed again."""
    width = layer.N // parts
    if perm.numel() != width:
        raise ValueError("the permutation must cover one block of columns")
    p = perm.long().to(layer.qweight.device)
    cols = torch.cat([p + b * width for b in range(parts)])
    z = unpack_fields(layer.qzeros.t().contiguous(), layer.bits)            # [N, G]
    qzeros = pack_fields_torch(z.index_select(0, cols).contiguous(), layer.bits).t().contiguous()
    return PackedLayer(layer.bits, layer.group_size, layer.K, layer.N, layer.qweight.index_select(1, cols).contiguous(),
                       qzeros, layer.scales.index_select(1, cols).contiguous(), layer.g_idx.clone(),
                       None if layer.bias is None else layer.bias.index_select(0, cols).contiguous())


def fold_act_order(consumer: PackedLayer, producer: PackedLayer, sorted_qweight: torch.Tensor, perm: torch.Tensor,
                   parts: int = 1) -> Tuple[PackedLayer, PackedLayer]:
    """Remove the act-order gather of ``consumer``, whose input is an element-wise function of ``producer``'s output
    (block by block for a fused producer of ``parts`` blocks).  ``perm`` is the stable argsort of the consumer's
    ``g_idx`` and ``sorted_qweight`` its rows in that order (``ops.sort_rows``); the consumer must have whole groups
    (every group exactly ``group_size`` rows), so that the sorted ``g_idx`` is ``k // group_size``.  Returns
    ``(consumer', producer')``: consumer' has ``g_idx == k // group_size`` and expects its input in sorted order,
    which producer' delivers because its output columns were re-ordered by ``perm``."""
    gs = _group_size(consumer)
    g_sorted = consumer.g_idx.long().index_select(0, perm.long())
    if not torch.equal(g_sorted, torch.arange(consumer.K, device=g_sorted.device) // gs):
        raise ValueError("the consumer's groups are not whole: sorting its rows does not give k // group_size")
    folded = PackedLayer(consumer.bits, consumer.group_size, consumer.K, consumer.N, sorted_qweight, consumer.qzeros,
                         consumer.scales, (torch.arange(consumer.K, device=g_sorted.device) // gs).to(torch.int32),
                         consumer.bias)
    return folded, permute_columns(producer, perm, parts)


def shard_column(layer: PackedLayer, rank: int, world: int, parts: int = 1,
                 sizes: Optional[Sequence[int]] = None) -> PackedLayer:
    """Column-parallel shard.  ``parts`` > 1: the layer is ``parts`` equal blocks side by side (q|k|v, gate|up) and
    the rank takes the same range of each.  ``sizes``: per-rank widths of one block (default: as even as possible
    in multiples of 32)."""
    if layer.N % parts:
        raise ValueError("the layer's width is not a multiple of the number of fused parts")
    width = layer.N // parts
    if sizes is None:
        sizes = split_sizes(width, world, 32)
    a, b = bounds(sizes, rank)
    if a == b:
        raise ValueError("more ranks than 32-column blocks")
    return take_columns(layer, [(p * width + a, p * width + b) for p in range(parts)])


def shard_row(layer: PackedLayer, rank: int, world: int,
              sizes: Optional[Sequence[int]] = None) -> Tuple[PackedLayer, Tuple[int, int]]:
    """Row-parallel shard and the range of input features ``[k_a, k_b)`` it consumes.  ``sizes``: per-rank row
    counts (default: whole groups, as even as possible, when the layer's ``g_idx`` is ``k // group_size``;
    multiples of 32 rows otherwise)."""
    gs = _group_size(layer)
    if sizes is None:
        unit = 32
        if is_trivial(layer) and layer.K % gs == 0:
            unit = gs if gs % 32 == 0 else gs * 32
            if layer.K % unit:
                unit = 32
        sizes = split_sizes(layer.K, world, unit)
    k_a, k_b = bounds(sizes, rank)
    if k_a == k_b:
        raise ValueError("more ranks than row blocks")
    return take_rows(layer, k_a, k_b, keep_bias=(rank == 0)), (k_a, k_b)


__all__ = ["split_sizes", "bounds", "is_trivial", "take_columns", "take_rows", "shard_column", "shard_row",
           "unpack_fields", "pack_fields_torch", "permute_columns", "fold_act_order"]
