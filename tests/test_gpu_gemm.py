"""GPU parity of the tcgen05 prefill dequant-GEMM against the CPU oracle (through the C ABI)."""
import numpy as np
import pytest
import torch

from oracle import gptq_oracle as O

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from autogptq.tvm_b200 import QuantLinear, ops, synth
    DEV = torch.device("cuda:0")


def _layer_np(layer):
    return (layer.qweight.numpy(), layer.qzeros.numpy(), layer.scales.numpy(), layer.g_idx.numpy())


def _check(y, x, W, bias=None):
    ref = O.forward_fp64(x, W, bias)
    got = y.detach().cpu().numpy().astype(np.float64)
    err = np.abs(got - ref)
    tol = O.output_tolerance(x, W)              # contract: 1e-2 * ||x||_2 * max|w| per output
    assert np.all(err <= tol), f"contract tolerance exceeded: {err.max()} > {tol.min()}"
    band = 2.0 ** -10 * np.abs(ref) + 0.02 * tol  # fp32 accumulation, one fp16 rounding
    assert np.all(err <= band), f"max err {err.max()} outside the fp32-accumulate band"


def _status_clear():
    ops.check_status(DEV)      # raises if a bounded wait of any kernel expired


GEMM_CASES = [
    # bits, K, N, gs, M, bias
    (4, 256, 128, 128, 16, False),
    (4, 512, 256, 128, 48, True),
    (4, 1024, 384, 64, 130, False),      # two M tiles per CTA, M tail
    (4, 352, 96, 32, 20, False),         # K tail (352 = 5.5 k-tiles), N < one tile
    (4, 4096, 1024, 128, 300, True),
    (3, 256, 128, 128, 16, False),
    (3, 1024, 256, 128, 77, True),
    (3, 4096, 512, 128, 200, False),
    (3, 352, 96, -1, 33, False),
    (4, 512, 128, 128, 1, False),        # works for any M >= 1
    (3, 2048, 19200, 128, 16, True),     # 150 column tiles: two CTAs (one group of weight warps each) per SM
    (4, 1024, 19200, 64, 40, False),     # the same with a 64-row tile of x
]


@pytest.mark.parametrize("bits,K,N,gs,M,bias", GEMM_CASES)
def test_gemm_vs_oracle(bits, K, N, gs, M, bias):
    if N == 19200:
        assert ops.gemm_split(M, K, N, bits)[1] == 2, "this case is meant to run two CTAs per SM"
    layer = synth.make_layer(bits, K, N, gs, False, bias=bias, seed=K + N + M)
    x = synth.make_x(M, K, seed=M)
    _, _, W = O.dequantize(*_layer_np(layer), bits)
    d = layer.to(DEV)
    y = ops.gemm(x.to(DEV), d.qweight, d.qzeros, d.scales, None, bits, gs, bias=d.bias)
    _check(y, x.numpy(), W, None if layer.bias is None else layer.bias.numpy())
    y2 = ops.gemm(x.to(DEV), d.qweight, d.qzeros, d.scales, d.g_idx, bits, gs, bias=d.bias)
    assert torch.equal(y, y2), "explicit k // group_size g_idx must give the same bits"
    _status_clear()


SPLIT_K_CASES = [
    # bits, K, N, gs, M, bias: few column tiles and a long K, so that several CTAs share one output tile
    (4, 4096, 1024, 128, 16, True),      # 8 column tiles, four runs of 16 k-tiles
    (3, 4096, 512, 128, 48, False),
    (4, 8192, 256, 128, 100, True),      # above 64 rows: three runs of unequal length (128 k-tiles)
    (4, 2112, 128, 32, 20, False),       # 33 k-tiles: runs of 16 and 17
    (3, 6144, 384, -1, 7, True),
]


@pytest.mark.parametrize("bits,K,N,gs,M,bias", SPLIT_K_CASES)
def test_gemm_with_k_split_over_ctas_vs_oracle(bits, K, N, gs, M, bias):
    """Up to 128 rows and fewer column tiles than SMs: K is cut into runs, one CTA per run, and the last CTA of a
    tile to finish sums the fp32 partial sums in run order.  Same oracle and tolerance as the unsplit kernel; the
    result must not depend on which CTA arrives last, and the tile counters must be back at zero for the next call."""
    assert ops.gemm_split(M, K, N, bits)[0] > 1, "this case is meant to run with K split over several CTAs"
    layer = synth.make_layer(bits, K, N, gs, False, bias=bias, seed=K + N + M)
    x = synth.make_x(M, K, seed=M)
    _, _, W = O.dequantize(*_layer_np(layer), bits)
    d = layer.to(DEV)
    xd = x.to(DEV)
    y = ops.gemm(xd, d.qweight, d.qzeros, d.scales, None, bits, gs, bias=d.bias)
    _check(y, x.numpy(), W, None if layer.bias is None else layer.bias.numpy())
    for _ in range(5):
        assert torch.equal(y, ops.gemm(xd, d.qweight, d.qzeros, d.scales, None, bits, gs, bias=d.bias))
    _status_clear()


@pytest.mark.parametrize("bits,K,N,gs,M", [(4, 1024, 256, 128, 40), (3, 1024, 256, 128, 150), (4, 512, 160, 64, 17)])
def test_gemm_act_order_through_quantlinear(bits, K, N, gs, M):
    layer = synth.make_layer(bits, K, N, gs, act_order=True, seed=3 * bits + M)
    _, _, W = O.dequantize(*_layer_np(layer), bits)
    mod = QuantLinear(bits, gs, K, N, False)
    mod.qweight, mod.qzeros, mod.scales, mod.g_idx = layer.qweight, layer.qzeros, layer.scales, layer.g_idx
    mod = mod.to(DEV)
    x = synth.make_x(M, K, seed=5)
    y = mod(x.to(DEV).reshape(1, M, K))
    assert tuple(y.shape) == (1, M, N)
    _check(y.reshape(M, N), x.numpy(), W)
    _status_clear()


@pytest.mark.parametrize("M", [16, 128])
def test_gemm_config2_vs_oracle(M):
    """4-bit, K=4096, N=12288 (fused QKV), the prefill configuration, at the sizes the oracle finishes quickly.
    16 rows run as three runs of K on two CTAs per SM, 128 rows as one CTA per column tile."""
    assert ops.gemm_split(M, 4096, 12288, 4) == ((3, 2) if M == 16 else (1, 1))
    layer = synth.make_layer(4, 4096, 12288, 128, False, seed=21)
    x = synth.make_x(M, 4096, seed=M)
    _, _, W = O.dequantize(*_layer_np(layer), 4)
    d = layer.to(DEV)
    y = ops.gemm(x.to(DEV), d.qweight, d.qzeros, d.scales, None, 4, 128)
    _check(y, x.numpy(), W)
    _status_clear()


@pytest.mark.parametrize("bits,M", [(4, 2048), (4, 512), (3, 512)])
def test_gemm_full_size_against_dequantised_product(bits, M):
    """At the full prefill sizes the check is a property: the fused kernel equals x @ W for the W that the
    (bit-exact, separately tested) dequantise kernel produces, evaluated by torch in fp32."""
    K, N = 4096, 12288
    d = synth.make_layer(bits, K, N, 128, False, seed=33, device=DEV)
    x = synth.make_x(M, K, seed=9, device=DEV)
    _, W = ops.dequantize(d.qweight, d.qzeros, d.scales, d.g_idx, bits, 128, want_q=False)
    y = ops.gemm(x, d.qweight, d.qzeros, d.scales, None, bits, 128)
    ref = x.float() @ W.float()
    err = (y.float() - ref).abs()
    tol = 1e-2 * x.float().norm(dim=1, keepdim=True) * W.float().abs().max()
    assert bool((err <= tol).all())
    assert bool((err <= 2.0 ** -10 * ref.abs() + 0.02 * tol).all())
    _status_clear()


def test_group_sizes_that_cut_through_row_blocks():
    """The tensor-core kernel takes one group per aligned 32-row block.  A layer with group size 16 must be refused
    by the entry point (not evaluated wrongly) and still run correctly through the module, which falls back to
    GEMV passes."""
    bits, K, N, gs, M = 4, 256, 128, 16, 16
    layer = synth.make_layer(bits, K, N, gs, False, seed=5)
    x = synth.make_x(M, K, seed=2)
    _, _, W = O.dequantize(*_layer_np(layer), bits)
    d = layer.to(DEV)
    with pytest.raises(RuntimeError, match="32-row"):
        ops.gemm(x.to(DEV), d.qweight, d.qzeros, d.scales, None, bits, gs)
    mod = QuantLinear(bits, gs, K, N, False)
    mod.qweight, mod.qzeros, mod.scales, mod.g_idx = layer.qweight, layer.qzeros, layer.scales, layer.g_idx
    mod = mod.to(DEV)
    _check(mod(x.to(DEV)), x.numpy(), W)
    assert mod._gemm_ok is False
