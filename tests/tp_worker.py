"""One rank of tests/test_gpu_tp.py (launched by torch.distributed.run)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    arch, fused_allreduce = sys.argv[1], int(sys.argv[2])
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
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
        print("TP_PARITY_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
