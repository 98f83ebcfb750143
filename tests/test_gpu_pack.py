"""GPU packing (b200gptq_pack_fields and QuantLinear.pack on a CUDA device) against the reference's own
pack outputs (tests/golden/pack_*.npz, produced by auto_gptq/nn_modules/qlinear.py:77-175) and against the
CPU packer of the module, bit for bit."""
import os

import numpy as np
import pytest
import torch
import torch.nn as nn

from conftest import GOLDEN_DIR, golden_files

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from autogptq.tvm_b200 import QuantLinear, ops
    from autogptq.tvm_b200.qlinear import _pack_fields
    DEV = torch.device("cuda:0")


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("R,C", [(32, 32), (128, 96), (4096, 1000)])
def test_pack_fields_equals_the_cpu_packer(bits, R, C):
    gen = torch.Generator().manual_seed(bits * 1000 + R + C)
    vals = torch.randint(0, 1 << bits, (R, C), generator=gen, dtype=torch.int64)
    # a few values wider than the field, and negative ones: the reference does not mask, neither do we
    vals[0, 0] = (1 << bits) + 1
    vals[R - 1, C - 1] = -1
    vals[R // 2, C // 2] = 0x12345678
    want = _pack_fields(torch.from_numpy(vals.numpy().astype(np.uint32).astype(np.int64)), bits)
    as_i32 = torch.from_numpy(vals.numpy().astype(np.uint32).view(np.int32).copy())
    got = ops.pack_fields(as_i32.to(DEV), bits)
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("fname", golden_files("pack_"))
def test_module_pack_on_gpu_matches_reference_vectors(fname):
    g = np.load(os.path.join(GOLDEN_DIR, fname))
    bits, gs = int(g["bits"]), int(g["group_size"])
    N, K = g["weight"].shape
    lin = nn.Linear(K, N, bias=True)
    lin.weight.data = torch.from_numpy(g["weight"])
    lin.bias.data = torch.from_numpy(g["lin_bias"])
    lin = lin.to(DEV)
    m = QuantLinear(bits, gs, K, N, True).to(DEV)
    m.pack(lin, torch.from_numpy(g["scales_in"]).to(DEV), torch.from_numpy(g["zeros_in"]).to(DEV),
           torch.from_numpy(g["g_idx"]).to(DEV))
    assert m.qweight.is_cuda and m.qzeros.is_cuda
    assert np.array_equal(m.qweight.cpu().numpy(), g["qweight"])
    assert np.array_equal(m.qzeros.cpu().numpy(), g["qzeros"])
    assert np.array_equal(m.scales.cpu().numpy().view(np.uint16), g["scales"].view(np.uint16))
    # and the packed layer computes what the reference computed with it
    y = m(torch.from_numpy(g["x"]).to(DEV))
    ref = g["out"].astype(np.float32)
    assert np.allclose(y.float().cpu().numpy(), ref, rtol=2e-3, atol=2e-3 * np.abs(ref).max())


def test_module_pack_gpu_equals_cpu_at_layer_size():
    bits, gs, K, N = 4, 128, 1024, 512
    gen = torch.Generator().manual_seed(5)
    lin = nn.Linear(K, N, bias=False)
    lin.weight.data = torch.randn(N, K, generator=gen) * 0.05
    G = K // gs
    scales = torch.rand(N, G, generator=gen) * 0.02 + 1e-3
    zeros = torch.randint(1, 16, (N, G), generator=gen).float()
    a = QuantLinear(bits, gs, K, N, False)
    a.pack(lin, scales, zeros)
    b = QuantLinear(bits, gs, K, N, False).to(DEV)
    b.pack(lin.to(DEV), scales.to(DEV), zeros.to(DEV))
    assert torch.equal(a.qweight, b.qweight.cpu())
    assert torch.equal(a.qzeros, b.qzeros.cpu())
    assert torch.equal(a.scales, b.scales.cpu())


def test_pack_fields_rejects_bad_arguments():
    with pytest.raises(ValueError):
        ops.pack_fields(torch.zeros((31, 8), dtype=torch.int32, device=DEV), 4)
    with pytest.raises(ValueError):
        ops.pack_fields(torch.zeros((32, 8), dtype=torch.int32, device=DEV), 5)
    with pytest.raises(RuntimeError):
        ops.pack_fields(torch.zeros((32, 8), dtype=torch.int32), 4)
