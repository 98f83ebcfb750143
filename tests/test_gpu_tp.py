"""Tensor parallelism on real GPUs: a decoder cut over two ranks (column-parallel q|k|v and gate|up, row-parallel
o_proj and down_proj, one all-reduce each) must compute the same logits as the same model on one GPU, within
the tolerance of the output contract applied to the vocabulary projection.  Needs two GPUs; skipped otherwise.
The ranks are child processes (one per GPU) that rendezvous on 127.0.0.1."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "tp_worker.py")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(*worker_args):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", env["MASTER_PORT"], WORKER, *map(str, worker_args)]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-4000:]
    assert "TP_WORKER_OK" in r.stdout, r.stdout[-4000:]


@pytest.mark.parametrize("arch", ["llama", "opt"])
@pytest.mark.parametrize("fused_allreduce", [0, 1])
def test_two_gpu_decoder_equals_single_gpu_decoder(arch, fused_allreduce):
    _run("decoder", arch, fused_allreduce)


def test_fused_allreduce_gemv_against_the_oracle_and_its_bounded_wait():
    """b200gptq_gemv_tp on two row shards gives the full layer's result (oracle, same tolerance as everywhere) with
    the same bits on both ranks; a peer that never joins makes the wait run out after the given number of cycles
    and the kernel report it instead of hanging."""
    _run("gemv")
