"""Tensor-parallel slicing rules, checked on CPU: two gloo ranks evaluate their shards with the CPU
oracle and exchange results with the collectives the GPU path uses (all-gather for column-parallel
outputs, all-reduce for row-parallel ones)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from autogptq.tvm_b200 import synth, tp
from oracle import gptq_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dense(layer):
    _, _, W = O.dequantize(layer.qweight.numpy(), layer.qzeros.numpy(), layer.scales.numpy(), layer.g_idx.numpy(),
                           layer.bits)
    return torch.from_numpy(W.astype(np.float32))


def _worker(rank, world, port, bits, K, N, gs):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    try:
        full = synth.make_layer(bits, K, N, gs, False, bias=True, seed=5)     # same seed on every rank
        x = synth.make_x(3, K, seed=2).float()
        want = x @ _dense(full) + full.bias.float()
        # column-parallel: concatenate the ranks' outputs
        col = tp.shard_column(full, rank, world)
        y_col = x @ _dense(col) + col.bias.float()
        sizes = tp.split_sizes(N, world, 32)
        parts = [torch.empty(3, s) for s in sizes]
        dist.all_gather(parts, y_col) if len(set(sizes)) == 1 else None
        if len(set(sizes)) != 1:  # uneven shards: gather through padded buffers
            pad = torch.zeros(3, max(sizes)); pad[:, :y_col.shape[1]] = y_col
            bufs = [torch.empty(3, max(sizes)) for _ in range(world)]
            dist.all_gather(bufs, pad)
            parts = [b[:, :s] for b, s in zip(bufs, sizes)]
        assert torch.allclose(torch.cat(parts, dim=1), want, atol=1e-4)
        # row-parallel: sum the ranks' outputs; only rank 0 carries the bias
        row, (k_a, k_b) = tp.shard_row(full, rank, world)
        assert (row.bias is not None) == (rank == 0)
        y_row = x[:, k_a:k_b] @ _dense(row) + (row.bias.float() if row.bias is not None else 0.0)
        dist.all_reduce(y_row)
        assert torch.allclose(y_row, want, atol=1e-3)
        # row-parallel on an act-order layer: every shard keeps the global group ids of its rows and the whole
        # scales / qzeros (W[k, n] = scales[g_idx[k], n] * (q[k, n] - zeros[g_idx[k], n]), qlinear.py:242)
        act = synth.make_layer(bits, K, N, gs, True, bias=False, seed=6)
        want_act = x @ _dense(act)
        row, (k_a, k_b) = tp.shard_row(act, rank, world)
        assert row.scales.shape == act.scales.shape and torch.equal(row.g_idx, act.g_idx[k_a:k_b])
        y_row = x[:, k_a:k_b] @ _dense(row)
        dist.all_reduce(y_row)
        assert torch.allclose(y_row, want_act, atol=1e-3)
        # a fused layer of three equal blocks (q|k|v): the rank owns the same columns of every block
        if N % 96 == 0:
            fused = tp.shard_column(full, rank, world, parts=3)
            a, b = tp.bounds(tp.split_sizes(N // 3, world, 32), rank)
            cols = torch.cat([torch.arange(p * (N // 3) + a, p * (N // 3) + b) for p in range(3)])
            assert torch.allclose(x @ _dense(fused) + fused.bias.float(), want[:, cols], atol=1e-4)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("bits,K,N,gs", [(4, 512, 128, 128), (3, 768, 192, 128), (4, 256, 64, 64)])
def test_two_rank_sharding_matches_the_full_layer(bits, K, N, gs):
    mp.spawn(_worker, args=(2, _free_port(), bits, K, N, gs), nprocs=2, join=True)


def test_split_sizes_and_errors():
    assert tp.split_sizes(11008, 8, 128) == [1408] * 6 + [1280] * 2
    assert sum(tp.split_sizes(4096, 8, 32)) == 4096
    with pytest.raises(ValueError):
        tp.split_sizes(100, 2, 32)
    act = synth.make_layer(4, 256, 64, 64, act_order=True, seed=1)
    shard, (k_a, k_b) = tp.shard_row(act, 1, 2)
    assert (k_a, k_b) == (128, 256) and shard.K == 128 and shard.scales.shape[0] == 4   # all groups stay
    with pytest.raises(ValueError):
        tp.take_rows(act, 16, 48, keep_bias=False)       # cuts must fall on multiples of 32 rows
    with pytest.raises(ValueError):
        tp.take_columns(act, [(0, 48)])                  # and on multiples of 32 columns


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_field_packing_round_trip(bits):
    w = torch.randint(-2**31, 2**31 - 1, (bits * 4, 40), dtype=torch.int64).to(torch.int32)
    f = tp.unpack_fields(w, bits)
    assert torch.equal(tp.pack_fields_torch(f, bits), w)
    if bits != 8:
        assert np.array_equal(f.numpy(), O.unpack_qweight(w.numpy(), bits).astype(np.int32))


@pytest.mark.parametrize("bits", [3, 4])
def test_act_order_fold_keeps_the_function(bits):
    """gate|up -> SiLU*up -> down with an act-order down projection: after the fold the down projection has
    g_idx == k // group_size and the pair computes what it computed before (oracle weights)."""
    K, I, N = 256, 512, 96
    prod = synth.make_layer(bits, K, 2 * I, 128, True, bias=True, seed=1)
    cons = synth.make_layer(bits, I, N, 128, True, bias=True, seed=2)
    x = synth.make_x(3, K, seed=1).float()

    def ffn(p, c):
        u = x @ _dense(p) + p.bias.float()
        return (torch.nn.functional.silu(u[:, :I]) * u[:, I:]) @ _dense(c) + c.bias.float()

    want = ffn(prod, cons)
    perm = torch.sort(cons.g_idx.long(), stable=True).indices
    q = tp.unpack_fields(cons.qweight, bits)
    qs = tp.pack_fields_torch(q.index_select(0, perm).contiguous(), bits)     # what ops.sort_rows does on the GPU
    c2, p2 = tp.fold_act_order(cons, prod, qs, perm, parts=2)
    assert tp.is_trivial(c2)
    assert torch.allclose(ffn(p2, c2), want, atol=1e-3)
