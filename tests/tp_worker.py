"""One rank of tests/test_gpu_tp.py (launched by torch.distributed.run): ``tp_worker.py <mode> [args]``."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def decoder_parity(dev, rank, arch, fused_allreduce):
    from autogptq.tvm_b200 import decoder
    if arch == "llama":
        cfg = decoder.DecoderConfig(arch="llama", layers=3, hidden=512, heads=4, inter=1024, vocab=2000, bits=4,
                                    group_size=128, desc_act=False, max_seq=64)
    else:   # act-order: the row-parallel shards keep global group ids
        cfg = decoder.DecoderConfig(arch="opt", layers=2, hidden=512, heads=4, inter=1024, vocab=2000, bits=3,
                                    group_size=128, desc_act=True, max_seq=64)
    prompt = torch.randint(0, cfg.vocab, (1, 16), generator=torch.Generator().manual_seed(5)).to(dev)
    res = decoder.tp_parity(cfg, prompt, dev, fused_allreduce=bool(fused_allreduce))
    if rank == 0:
        print("parity", res, flush=True)
        assert res["ok"], res


def gemv_tp_cases(dev, rank, world):
    """b200gptq_gemv_tp on row shards against the CPU oracle's full layer."""
    from autogptq.tvm_b200 import ops, synth, tp
    from autogptq.tvm_b200.exchange import PeerExchange
    from oracle import gptq_oracle as O
    ex = PeerExchange(dev)
    cases = [  # bits, K, N, gs, act_order, bias, M
        (4, 1024, 512, 128, False, True, 1),      # streaming kernel, exchange inside its combine step
        (3, 2048, 1056, 128, False, False, 4),    # ragged last column group
        (4, 4096, 4096, 128, False, True, 8),
        (4, 1024, 512, 128, False, False, 1),     # the same shape again: counters keep counting
        (3, 1024, 288, 128, True, True, 2),       # act-order shard: general kernel + exchange kernel
    ]
    for bits, K, N, gs, act, bias, M in cases:
        full = synth.make_layer(bits, K, N, gs, act, bias=bias, seed=K + N + M)
        x = synth.make_x(M, K, seed=M)
        _, _, W = O.dequantize(full.qweight.numpy(), full.qzeros.numpy(), full.scales.numpy(), full.g_idx.numpy(), bits)
        ref = O.forward_fp64(x.numpy(), W, None if full.bias is None else full.bias.numpy())
        tol = O.output_tolerance(x.numpy(), W)
        shard, (k_a, k_b) = tp.shard_row(full, rank, world)
        d = shard.to(dev)
        g = None if tp.is_trivial(shard) else d.g_idx
        fb = None if full.bias is None else full.bias.to(dev)
        xs = x[:, k_a:k_b].contiguous().to(dev)
        for rep in range(2):   # twice in a row: both data slots, growing counters
            y = ops.gemv_tp(xs, d.qweight, d.qzeros, d.scales, g, bits, gs, ex, bias=fb)
            err = np.abs(y.cpu().numpy().astype(np.float64) - ref)
            assert np.all(err <= tol), (bits, K, N, act, M, rep, float(err.max()), float(tol.min()))
            band = 2.0 ** -9 * np.abs(ref) + 0.05 * tol
            assert np.all(err <= band), (bits, K, N, act, M, rep, float(err.max()))
        gathered = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(gathered, y)
        assert all(torch.equal(gathered[0], t) for t in gathered), "every rank must hold the same bits"
    assert ex.status() == 0
    # latency of one exchange of [1, 4096] (printed for the record; no assertion on a shared machine)
    y = torch.ones((1, 4096), dtype=torch.float16, device=dev)
    for _ in range(20):
        ops.tp_allreduce(y.fill_(1.0), ex)
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(200):
        ops.tp_allreduce(y, ex)
    e1.record()
    torch.cuda.synchronize()
    if rank == 0:
        print(f"exchange latency [1, 4096] x {world} ranks: {e0.elapsed_time(e1) * 1e3 / 200:.2f} us per call", flush=True)
    assert ex.status() == 0
    return ex


def timeout_case(dev, rank, ex):
    """A peer that never joins: rank 1 skips the call, rank 0's wait runs out after ~1 ms, the kernel raises the
    status word and returns; the process stays usable.  (Made on the host; nothing hangs or faults.)"""
    from autogptq.tvm_b200 import ops
    dist.barrier()
    if rank == 0:
        ex.timeout_cycles = 2_000_000
        y = torch.ones((1, 512), dtype=torch.float16, device=dev)
        ops.tp_allreduce(y, ex)
        assert ex.status() == 2, "the expired wait must be reported"
        z = torch.ones(4, device=dev) * 2          # the context still works
        assert float(z.sum()) == 8.0
    dist.barrier()


def main():
    mode = sys.argv[1]
    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    if mode == "decoder":
        decoder_parity(dev, rank, sys.argv[2], int(sys.argv[3]))
    elif mode == "gemv":
        ex = gemv_tp_cases(dev, rank, world)
        timeout_case(dev, rank, ex)    # last: it leaves the two ranks' counters apart
    else:
        raise SystemExit(f"unknown mode {mode}")
    dist.barrier()
    if rank == 0:
        print("TP_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
