"""The CPU oracle against the golden vectors that the reference itself produced
(tests/golden/make_golden.py), and against the live reference when it is present."""
import contextlib
import importlib.util
import io
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR, golden_files
from oracle import gptq_oracle as O


def _load(name):
    return dict(np.load(os.path.join(GOLDEN_DIR, name)))


def _same_fp16(a, b):
    """Bit equality of two fp16 arrays, with +0 and -0 identified."""
    a = np.asarray(a, np.float16) + np.float16(0)
    b = np.asarray(b, np.float16) + np.float16(0)
    return np.array_equal(a.view(np.uint16), b.view(np.uint16))


@pytest.mark.parametrize("fname", golden_files("forward_"))
def test_dequantize_bit_exact_vs_reference_vectors(fname):
    g = _load(fname)
    bits = int(g["bits"])
    q, z, W = O.dequantize(g["qweight"], g["qzeros"], g["scales"], g["g_idx"], bits)
    assert W.dtype == np.float16 and W.shape == g["W"].shape
    assert _same_fp16(W, g["W"])
    maxq = 2**bits - 1
    assert q.min() >= 0 and q.max() <= maxq
    assert z.min() >= 1 and z.max() <= maxq + 1


@pytest.mark.parametrize("fname", golden_files("forward_"))
def test_torch_oracle_forward_equals_reference_vectors(fname):
    g = _load(fname)
    bits = int(g["bits"])
    torch.set_num_threads(1)
    bias = g["bias"] if g["bias"].size else None
    orc = O.TorchQuantLinearOracle(bits, g["qweight"], g["qzeros"], g["scales"], g["g_idx"], bias)
    assert _same_fp16(orc.dequantize().numpy(), g["W"])
    out = orc.forward(torch.from_numpy(g["x"])).numpy()
    # the same torch build and thread count reproduce the stored fp16 matmul exactly;
    # another host may round the last bit differently, so also accept the contract's band
    ref64 = O.forward_fp64(g["x"], g["W"], bias)
    tol = O.output_tolerance(g["x"], g["W"])
    assert np.all(np.abs(out.astype(np.float64) - ref64) <= tol)
    assert np.all(np.abs(g["out"].astype(np.float64) - ref64) <= tol)
    assert np.max(np.abs(out.astype(np.float32) - g["out"].astype(np.float32))) <= 2e-2


@pytest.mark.parametrize("fname", golden_files("pack_"))
def test_pack_bit_exact_vs_reference_vectors(fname):
    g = _load(fname)
    bits = int(g["bits"])
    qweight, qzeros, scales = O.pack(g["weight"], g["scales_in"], g["zeros_in"], g["g_idx"], bits)
    assert np.array_equal(qweight, g["qweight"])
    assert np.array_equal(qzeros, g["qzeros"])
    assert _same_fp16(scales, g["scales"])


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_pack_unpack_round_trip(bits):
    rng = np.random.default_rng(bits)
    K, N = 128, 64
    vals = rng.integers(0, 2**bits, size=(K, N), dtype=np.uint32)
    words = O._pack_stream(vals, bits)
    assert words.shape == (K // 32 * bits, N)
    assert np.array_equal(O._unpack_stream(words, bits).astype(np.uint32), vals)


def test_known_answer_closed_form():
    """Parametric known-answer input used by the reference's hand-run scripts
    (pycuda_warpper.py:330-343): w = arange % 4, x = ones, scale = 1, zero = 0."""
    for bits in (3, 4):
        K, N = 256, 64
        w = (np.arange(N * K, dtype=np.int64) % 4).reshape(N, K).astype(np.float32)
        scales = np.ones((N, 1), np.float32)
        zeros = np.ones((N, 1), np.float32)  # zero-point 1 => stored field 0
        g_idx = np.zeros(K, np.int32)
        qweight, qzeros, s16 = O.pack(w, scales, zeros, g_idx, bits)  # q = w + zero = w + 1, z = 1
        q, z, W = O.dequantize(qweight, qzeros, s16, g_idx, bits)
        assert np.array_equal(W.astype(np.float32), w.T)
        out = O.forward_fp64(np.ones((1, K), np.float16), W)
        assert np.array_equal(out[0], w.sum(axis=1))


def test_zero_point_plus_one_is_not_masked():
    qzeros = np.full((1, 1), -1, np.int32)  # every 4-bit field = 15
    z = O.unpack_qzeros(qzeros, 4)
    assert z.shape == (1, 8) and np.all(z == 16)
    z3 = O.unpack_qzeros(np.full((1, 3), -1, np.int32), 3)
    assert z3.shape == (1, 32) and np.all(z3 == 8)


# The live reference: a checkout named by the environment, else the file staged by oracle/stage_ref.py.
REF_ROOT = os.environ.get("B200GPTQ_REFERENCE", os.environ.get("GPTQ_REFERENCE_ROOT", ""))
_STAGED = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "qlinear.py")
REF_FILE = os.path.join(REF_ROOT, "auto_gptq/nn_modules/qlinear.py") if REF_ROOT else _STAGED


@pytest.mark.skipif(not os.path.isfile(REF_FILE), reason="no reference checkout named and nothing staged")
@pytest.mark.parametrize("bits,K,N,gs,act", [(4, 1024, 256, 128, False), (3, 1024, 256, 128, True),
                                             (4, 512, 128, 32, True), (3, 512, 96, -1, False)])
def test_oracle_equals_live_reference(bits, K, N, gs, act):
    spec = importlib.util.spec_from_file_location("_ref_qlinear", REF_FILE)
    ref = importlib.util.module_from_spec(spec)
    with contextlib.redirect_stdout(io.StringIO()):
        spec.loader.exec_module(ref)
    gen = torch.Generator().manual_seed(bits * 1000 + K + N)
    layer = ref.QuantLinear(bits, gs, K, N, False)
    G = layer.scales.shape[0]
    layer.qweight = torch.randint(-2**31, 2**31 - 1, layer.qweight.shape, generator=gen).to(torch.int32)
    layer.qzeros = torch.randint(-2**31, 2**31 - 1, layer.qzeros.shape, generator=gen).to(torch.int32)
    layer.scales = (torch.randn(G, N, generator=gen).abs() * 0.02 + 1e-3).half()
    if act:
        layer.g_idx = (torch.randperm(K, generator=gen) // (gs if gs != -1 else K)).to(torch.int32)
    x = torch.randn(2, K, generator=gen).half()
    torch.set_num_threads(1)
    with contextlib.redirect_stdout(io.StringIO()):
        out_ref = layer.forward(x)
        W_ref = layer.forward(torch.eye(K, dtype=torch.float16))
    orc = O.TorchQuantLinearOracle(bits, layer.qweight, layer.qzeros, layer.scales, layer.g_idx)
    _, _, W = O.dequantize(layer.qweight, layer.qzeros, layer.scales, layer.g_idx, bits)
    assert _same_fp16(W, W_ref.numpy())
    assert _same_fp16(orc.dequantize().numpy(), W_ref.numpy())
    assert torch.equal(orc.forward(x), out_ref)
