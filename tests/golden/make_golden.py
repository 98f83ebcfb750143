"""Generate the golden vectors in this directory by RUNNING THE REFERENCE ITSELF.

Usage (only where the reference tree is available)::

    python tests/golden/make_golden.py /path/to/AutoGPTQ.tvm

The reference module ``auto_gptq/nn_modules/qlinear.py`` is loaded by file path
(the ``auto_gptq`` package itself needs ``accelerate``, which is not installed) and
its own ``QuantLinear.pack`` / ``QuantLinear.forward`` produce every expected
value stored here.  Nothing in this script computes an expected value by other
means.  The dequantised weight matrix is read out of the reference by pushing an
identity matrix through ``forward`` (``eye(K) @ W == W`` exactly in fp16).

Outputs: ``forward_*.npz`` (packed buffers, x, out, W) and ``pack_*.npz`` (float
weight, scales, zeros, g_idx and the packed result).
"""
import contextlib
import importlib.util
import io
import os
import sys

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    path = os.path.join(root, "auto_gptq", "nn_modules", "qlinear.py")
    spec = importlib.util.spec_from_file_location("_ref_qlinear", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def quiet(fn, *a, **kw):
    with contextlib.redirect_stdout(io.StringIO()):
        return fn(*a, **kw)


def rand_packed(gen, bits, K, N, G):
    qweight = torch.randint(-2**31, 2**31 - 1, (K // 32 * bits, N), generator=gen, dtype=torch.int64).to(torch.int32)
    qzeros = torch.randint(-2**31, 2**31 - 1, (G, N // 32 * bits), generator=gen, dtype=torch.int64).to(torch.int32)
    scales = (torch.randn(G, N, generator=gen).abs() * 0.02 + 1e-3).half()
    return qweight, qzeros, scales


FORWARD_CASES = [
    # name, bits, K, N, group_size, act_order, M, bias
    ("b4_g128", 4, 512, 64, 128, False, 1, False),
    ("b4_g64_act", 4, 256, 96, 64, True, 5, True),
    ("b4_perchannel", 4, 256, 32, -1, False, 3, False),
    ("b3_g128", 3, 512, 64, 128, False, 1, False),
    ("b3_g128_act", 3, 512, 96, 128, True, 4, True),
    ("b3_perchannel", 3, 256, 32, -1, False, 2, False),
    ("b2_g64", 2, 256, 64, 64, False, 2, True),
    ("b8_g128_act", 8, 256, 64, 128, True, 3, False),
    ("b4_ragged_group", 4, 320, 64, 128, False, 2, False),
]


def make_forward(ref, name, bits, K, N, gs, act, M, bias, seed):
    gen = torch.Generator().manual_seed(seed)
    layer = ref.QuantLinear(bits, gs, K, N, bias)
    G = layer.scales.shape[0]
    qweight, qzeros, scales = rand_packed(gen, bits, K, N, G)
    layer.qweight, layer.qzeros, layer.scales = qweight, qzeros, scales
    if act:
        group = gs if gs != -1 else K
        layer.g_idx = (torch.randperm(K, generator=gen) // group).to(torch.int32)
    if bias:
        layer.bias = torch.randn(N, generator=gen).half()
    x = torch.randn(M, K, generator=gen).half()
    out = quiet(layer.forward, x)
    saved_bias, layer.bias = layer.bias, None
    W = quiet(layer.forward, torch.eye(K, dtype=torch.float16))
    layer.bias = saved_bias
    np.savez_compressed(
        os.path.join(HERE, f"forward_{name}.npz"),
        bits=bits, group_size=gs,
        qweight=qweight.numpy(), qzeros=qzeros.numpy(), scales=scales.numpy(),
        g_idx=layer.g_idx.numpy(), x=x.numpy(), out=out.numpy(), W=W.numpy(),
        bias=(layer.bias.numpy() if bias else np.zeros(0, np.float16)),
    )


PACK_CASES = [
    ("b4_g64", 4, 128, 64, 64, False),
    ("b3_g64_act", 3, 128, 64, 64, True),
    ("b2_g32", 2, 64, 32, 32, False),
    ("b8_perchannel", 8, 64, 32, -1, False),
]


def make_pack(ref, name, bits, K, N, gs, act, seed):
    gen = torch.Generator().manual_seed(seed)
    lin = nn.Linear(K, N, bias=True)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(N, K, generator=gen) * 0.05)
        lin.bias.copy_(torch.randn(N, generator=gen) * 0.1)
    group = gs if gs != -1 else K
    G = K // group
    maxq = 2**bits - 1
    if act:
        g_idx = (torch.randperm(K, generator=gen) // group).to(torch.int32)
    else:
        g_idx = (torch.arange(K) // group).to(torch.int32)
    # asymmetric min/max grid per (output channel, group), as a GPTQ quantizer would emit
    Wt = lin.weight.data
    scales = torch.empty(N, G)
    zeros = torch.empty(N, G)
    for g in range(G):
        cols = (g_idx == g).nonzero().flatten()
        wmin = Wt[:, cols].min(1).values.clamp(max=0)
        wmax = Wt[:, cols].max(1).values.clamp(min=0)
        scales[:, g] = (wmax - wmin) / maxq
        zeros[:, g] = torch.round(-wmin / scales[:, g])
    layer = ref.QuantLinear(bits, gs, K, N, True)
    quiet(layer.pack, lin, scales.clone(), zeros.clone(), g_idx.clone())
    x = torch.randn(3, K, generator=gen).half()
    with torch.no_grad():
        out = quiet(layer.forward, x)
    np.savez_compressed(
        os.path.join(HERE, f"pack_{name}.npz"),
        bits=bits, group_size=gs,
        weight=lin.weight.data.numpy(), lin_bias=lin.bias.data.numpy(),
        scales_in=scales.numpy(), zeros_in=zeros.numpy(), g_idx=g_idx.numpy(),
        qweight=layer.qweight.numpy(), qzeros=layer.qzeros.numpy(),
        scales=layer.scales.numpy(), bias=layer.bias.detach().numpy(), x=x.numpy(), out=out.numpy(),
    )


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("GPTQ_REFERENCE_ROOT", "")
    if not os.path.isdir(root):
        raise SystemExit("give the path of the reference checkout")
    ref = load_reference(root)
    torch.set_num_threads(1)  # one thread => the stored fp16 matmul results do not depend on the host
    for i, case in enumerate(FORWARD_CASES):
        make_forward(ref, *case, seed=1000 + i)
    for i, case in enumerate(PACK_CASES):
        make_pack(ref, *case, seed=2000 + i)
    print("wrote", len(FORWARD_CASES) + len(PACK_CASES), "files to", HERE)


if __name__ == "__main__":
    main()
