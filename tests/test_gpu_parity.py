"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle.

Integer fields and dequantised fp16 weights must match bit for bit; outputs must
lie within ``1e-2 * ||x||_2 * max|w|`` of an fp64 product of the same dequantised
weights (the contract), and additionally within a much tighter band that an
fp32-accumulating kernel with an fp16 result is expected to meet.
"""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR, golden_files
from oracle import gptq_oracle as O

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from autogptq.tvm_b200 import QuantLinear, ops, synth, _lib
    DEV = torch.device("cuda:0")


def _bits16(a):
    return (np.asarray(a, np.float16) + np.float16(0)).view(np.uint16)


def _check_output(y, x, W, bias=None, tight=True):
    ref = O.forward_fp64(x, W, bias)
    got = y.detach().cpu().numpy().astype(np.float64).reshape(ref.shape)
    err = np.abs(got - ref)
    tol = O.output_tolerance(x, W)  # contract: 1e-2 * ||x||_2 * max|w| per output
    assert np.all(err <= tol), f"contract tolerance exceeded: max err {err.max()} tol {tol.min()}"
    if tight:
        # fp32 accumulation + one fp16 rounding of the result
        band = 2.0 ** -10 * np.abs(ref) + 0.05 * tol
        assert np.all(err <= band), f"max err {err.max()} exceeds the fp32-accumulate band"


def _layer_np(layer):
    return (layer.qweight.cpu().numpy(), layer.qzeros.cpu().numpy(), layer.scales.cpu().numpy(),
            layer.g_idx.cpu().numpy())


def test_library_is_loaded_from_the_tree():
    assert os.path.isfile(_lib.LIB_PATH)
    assert _lib.lib.b200gptq_abi_version() >= 1


@pytest.mark.parametrize("fname", golden_files("forward_"))
def test_dequant_bit_exact_on_reference_vectors(fname):
    g = dict(np.load(os.path.join(GOLDEN_DIR, fname)))
    bits, gs = int(g["bits"]), int(g["group_size"])
    t = lambda a: torch.from_numpy(a).to(DEV)
    q, W = ops.dequantize(t(g["qweight"]), t(g["qzeros"]), t(g["scales"]), t(g["g_idx"]), bits, gs,
                          want_q=(bits != 8))
    assert np.array_equal(_bits16(W.cpu().numpy()), _bits16(g["W"]))
    if bits != 8:
        assert np.array_equal(q.cpu().numpy(), O.unpack_qweight(g["qweight"], bits))


@pytest.mark.parametrize("bits,K,N,gs,act", [
    (4, 1024, 512, 128, False), (3, 1024, 512, 128, True), (4, 2048, 1056, 64, True),
    (3, 512, 96, -1, False), (2, 256, 64, 32, True), (8, 256, 96, 128, False), (4, 32, 32, 32, False),
])
def test_dequant_bit_exact_seeded(bits, K, N, gs, act):
    layer = synth.make_layer(bits, K, N, gs, act, seed=bits * 100 + N)
    q_ref, z_ref, W_ref = O.dequantize(*_layer_np(layer), bits)
    d = layer.to(DEV)
    q, W = ops.dequantize(d.qweight, d.qzeros, d.scales, d.g_idx, bits, gs, want_q=(bits != 8))
    assert np.array_equal(_bits16(W.cpu().numpy()), _bits16(W_ref))
    if bits != 8:
        assert np.array_equal(q.cpu().numpy(), q_ref)
    # g_idx = NULL means k // group_size
    if not act:
        _, W2 = ops.dequantize(d.qweight, d.qzeros, d.scales, None, bits, gs, want_q=False)
        assert torch.equal(W2, W)


@pytest.mark.parametrize("fname", golden_files("forward_"))
def test_quantlinear_forward_on_reference_vectors(fname):
    g = dict(np.load(os.path.join(GOLDEN_DIR, fname)))
    bits, gs = int(g["bits"]), int(g["group_size"])
    K, N = g["W"].shape
    has_bias = g["bias"].size > 0
    layer = QuantLinear(bits, gs, K, N, has_bias)
    layer.qweight = torch.from_numpy(g["qweight"])
    layer.qzeros = torch.from_numpy(g["qzeros"])
    layer.scales = torch.from_numpy(g["scales"])
    layer.g_idx = torch.from_numpy(g["g_idx"])
    if has_bias:
        layer.bias = torch.from_numpy(g["bias"])
    layer = layer.to(DEV)
    y = layer(torch.from_numpy(g["x"]).to(DEV))
    assert y.dtype == torch.float16 and tuple(y.shape) == g["out"].shape
    _check_output(y, g["x"], g["W"], g["bias"] if has_bias else None)
    # and close to what the reference itself returned (its fp16 matmul rounds differently)
    got, want = y.cpu().numpy().astype(np.float32), g["out"].astype(np.float32)
    assert np.all(np.abs(got - want) <= 2.0 ** -9 * np.abs(want) + 3e-2)


GEMV_CASES = [
    # bits, K, N, gs, act, bias
    (4, 1024, 512, 128, False, False),
    (4, 4096, 4096, 128, False, False),       # config 0
    (3, 4096, 11008, 128, True, False),       # config 1
    (3, 1024, 512, 128, False, True),
    (4, 2048, 1056, 64, True, True),          # N not a multiple of the strip width
    (4, 11008, 4096, 128, False, False),      # Llama down_proj
    (3, 512, 96, -1, False, False),
    (2, 256, 64, 32, True, False),
    (8, 256, 96, 128, False, True),
    (4, 32, 32, 32, False, False),            # smallest legal layer
]


def _trivial_g_idx(layer):
    gs = layer.group_size if layer.group_size != -1 else layer.K
    return bool(torch.equal(layer.g_idx.long(), torch.arange(layer.K) // gs))


@pytest.mark.parametrize("bits,K,N,gs,act,bias", GEMV_CASES)
@pytest.mark.parametrize("M", [1, 2, 5, 8])
@pytest.mark.parametrize("explicit_g_idx", [False, True])
def test_gemv_vs_oracle(bits, K, N, gs, act, bias, M, explicit_g_idx):
    """``explicit_g_idx=False`` passes NULL for layers whose g_idx is k // group_size, which is the contract
    of the streaming kernel; ``True`` always passes the tensor, which selects the general kernel.  Each
    case asserts which kernel it ran."""
    if M not in (1, 8) and K * N > 4096 * 4096:
        pytest.skip("large shapes are covered at M = 1 and 8")
    layer = synth.make_layer(bits, K, N, gs, act, bias=bias, seed=K + N + bits)
    if not explicit_g_idx and not _trivial_g_idx(layer):
        pytest.skip("an act-order g_idx cannot be passed as NULL (the sorted-rows test covers that route)")
    x = synth.make_x(M, K, seed=M)
    _, _, W = O.dequantize(*_layer_np(layer), bits)
    d = layer.to(DEV)
    g = d.g_idx if explicit_g_idx else None
    path = _lib.gemv_path(M, K, N, bits, gs, g is not None)
    streams = (not explicit_g_idx) and bits in (3, 4) and K % 128 == 0 and (gs == -1 or gs % 128 == 0)
    assert path == (_lib.PATH_STREAM if streams else _lib.PATH_GENERIC)
    y = ops.gemv(x.to(DEV), d.qweight, d.qzeros, d.scales, g, bits, gs, bias=d.bias)
    _check_output(y, x.numpy(), W, None if layer.bias is None else layer.bias.numpy())
    y2 = ops.gemv(x.to(DEV), d.qweight, d.qzeros, d.scales, g, bits, gs, bias=d.bias)
    assert torch.equal(y, y2), "two runs on the same inputs must agree bit for bit"


STREAM_CASES = [
    # bits, K, N, gs, bias : shapes that stress the streaming kernel's work split
    (4, 4096, 4096, 128, True),          # config 0 with bias through the pushed combine
    (3, 4096, 11008, 128, False),        # config-1 shape without act-order: uneven K split (32 units over 6 CTAs)
    (4, 11008, 4096, 128, False),        # 86 units per column group
    (3, 11008, 4096, 128, True),
    (4, 1024, 1056, 128, True),          # N not a multiple of 256 with clusters > 1
    (3, 2048, 2080, 256, False),         # group of two units, ragged last column group
    (4, 8192, 512, 1024, False),         # few column groups, long slices, groups of 8 units
    (3, 36864, 1024, 128, False),        # slices longer than the ring and than one stage of x
    (4, 1536, 256, -1, False),           # one group over all rows
    (3, 128, 32, 128, False),            # one unit, one column chunk
]


@pytest.mark.parametrize("bits,K,N,gs,bias", STREAM_CASES)
@pytest.mark.parametrize("M", [1, 3, 8])
def test_streaming_gemv_vs_oracle(bits, K, N, gs, bias, M):
    layer = synth.make_layer(bits, K, N, gs, False, bias=bias, seed=3 * K + N + bits)
    x = synth.make_x(M, K, seed=10 + M)
    _, _, W = O.dequantize(*_layer_np(layer), bits)
    d = layer.to(DEV)
    assert _lib.gemv_path(M, K, N, bits, gs, False) == _lib.PATH_STREAM
    y = ops.gemv(x.to(DEV), d.qweight, d.qzeros, d.scales, None, bits, gs, bias=d.bias)
    _check_output(y, x.numpy(), W, None if layer.bias is None else layer.bias.numpy())
    y2 = ops.gemv(x.to(DEV), d.qweight, d.qzeros, d.scales, None, bits, gs, bias=d.bias)
    assert torch.equal(y, y2)


SINGLE_ROW_CASES = [
    # bits, K, N, gs, act, bias : one row of x; the 3-bit ones run on the integer tensor path (x in fixed point per
    # 128 rows of K, four byte planes), the 4-bit ones on fp16 fragments
    (3, 4096, 11008, 128, True, False),      # config 1
    (3, 4096, 11008, 128, False, True),
    (4, 4096, 12288, 128, True, False),      # fused q|k|v
    (3, 8192, 8192, 1024, True, True),       # groups of 8 units
    (3, 2048, 6400, -1, False, True),        # one group over all rows
    (3, 1152, 3584, 128, True, False),       # 9 units
    (3, 128, 8192, 128, False, True),        # one unit
    (3, 36864, 512, 128, True, False),       # slices longer than one stage of x, through a gather
]


@pytest.mark.parametrize("bits,K,N,gs,act,bias", SINGLE_ROW_CASES)
def test_single_row_gemv_vs_oracle(bits, K, N, gs, act, bias):
    layer = synth.make_layer(bits, K, N, gs, act, bias=bias, seed=7 * K + N + bits)
    x = synth.make_x(1, K, seed=21)
    _, _, W = O.dequantize(*_layer_np(layer), bits)
    d = layer.to(DEV)
    if act:
        qw, perm, _ = ops.sort_rows(d.qweight, d.g_idx, bits)
    else:
        qw, perm = d.qweight, None
    assert _lib.gemv_path(1, K, N, bits, gs, False) == _lib.PATH_STREAM
    b = None if layer.bias is None else layer.bias.numpy()
    y = ops.gemv(x.to(DEV), qw, d.qzeros, d.scales, None, bits, gs, x_perm=perm, bias=d.bias)
    _check_output(y, x.numpy(), W, b)
    assert torch.equal(y, ops.gemv(x.to(DEV), qw, d.qzeros, d.scales, None, bits, gs, x_perm=perm, bias=d.bias))
    plan = ops.GemvPlan(qw, d.qzeros, d.scales, None, perm, d.bias, 1, bits, gs)
    assert torch.equal(plan.run(x.to(DEV)), y)
    _check_output(ops.gemv(x.to(DEV), qw, d.qzeros, d.scales, None, bits, gs, x_perm=perm, bias=d.bias, tuning=(2, 3)),
                  x.numpy(), W, b)
    ops.check_status(DEV)


def test_single_row_value_ranges():
    """On the integer tensor path x is converted to fixed point per 128 rows of K: rows of zeros, a wide dynamic
    range inside a unit, values at the ends of the fp16 range and a NaN must all come out as fp32 accumulation
    would give them."""
    bits, K, N, gs = 3, 4096, 4736, 128
    layer = synth.make_layer(bits, K, N, gs, False, seed=99)
    _, _, W = O.dequantize(*_layer_np(layer), bits)
    d = layer.to(DEV)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1, K)).astype(np.float32)
    x[0, 128:256] = 0.0                                            # a unit of zeros
    x[0, 256:384] *= np.logspace(-7, 0, 128, dtype=np.float32)    # 2^-23 .. 1 inside one unit
    x[0, 384:512] *= 2.0 ** -20                                    # a unit of fp16 subnormals
    x[0, 512] = 3.0e4                                              # near the top of the range
    x[0, 640:768] = 0.0
    x[0, 700] = 6.0e-8                                             # the smallest subnormal alone in its unit
    xh = torch.from_numpy(x).to(torch.float16)
    y = ops.gemv(xh.to(DEV), d.qweight, d.qzeros, d.scales, None, bits, gs)
    _check_output(y, xh.numpy(), W)
    xh[0, 1000] = float("nan")
    y = ops.gemv(xh.to(DEV), d.qweight, d.qzeros, d.scales, None, bits, gs)
    assert bool(torch.isnan(y).all())


@pytest.mark.parametrize("bits,K,N,gs,act,M", [(4, 4096, 4096, 128, False, 1), (3, 2048, 1056, 128, False, 5),
                                               (4, 512, 96, 64, True, 2), (8, 256, 96, 128, False, 8)])
def test_prepared_plan_equals_the_stateless_call(bits, K, N, gs, act, M):
    """b200gptq_gemv_plan_* (one launch per call, descriptors built once) against b200gptq_gemv and
    b200gptq_gemv_tuned with other tuning parameters: same bits, and the plan can be run repeatedly."""
    layer = synth.make_layer(bits, K, N, gs, act, bias=True, seed=K + M).to(DEV)
    g = layer.g_idx if act else None
    x = synth.make_x(M, K, seed=M, device=DEV)
    want = ops.gemv(x, layer.qweight, layer.qzeros, layer.scales, g, bits, gs, bias=layer.bias)
    plan = ops.GemvPlan(layer.qweight, layer.qzeros, layer.scales, g, None, layer.bias, M, bits, gs)
    for _ in range(3):
        assert torch.equal(plan.run(x), want)
    tuned = ops.gemv(x, layer.qweight, layer.qzeros, layer.scales, g, bits, gs, bias=layer.bias, tuning=(2, 3))
    # a different K split sums in a different order: equal within the tolerance, not necessarily bit for bit
    _check_output(tuned, x.cpu().numpy(), O.dequantize(*_layer_np(layer.to("cpu")), bits)[2], layer.bias.cpu().numpy())
    with pytest.raises(ValueError):
        plan.run(x[:, :K // 2].contiguous())
    del plan


@pytest.mark.parametrize("bits,K,N,gs", [(4, 4096, 4096, 128), (3, 4096, 11008, 128), (4, 1024, 544, 64)])
@pytest.mark.parametrize("M", [1, 4])
def test_sorted_rows_path_matches_oracle(bits, K, N, gs, M):
    """Act-order layer evaluated through QuantLinear: rows re-ordered by group, x gathered."""
    layer = synth.make_layer(bits, K, N, gs, act_order=True, seed=11 + bits)
    _, _, W = O.dequantize(*_layer_np(layer), bits)
    d = layer.to(DEV)
    qs, perm, g_sorted = ops.sort_rows(d.qweight, d.g_idx, bits)
    assert torch.equal(g_sorted, d.g_idx[perm.long()])
    assert bool((g_sorted[1:] >= g_sorted[:-1]).all())
    _, Ws = ops.dequantize(qs, d.qzeros, d.scales, g_sorted, bits, gs, want_q=False)
    assert np.array_equal(_bits16(Ws.cpu().numpy()), _bits16(W[perm.cpu().numpy()]))
    x = synth.make_x(M, K, seed=3)
    y = ops.gemv(x.to(DEV), qs, d.qzeros, d.scales, g_sorted, bits, gs, x_perm=perm)
    _check_output(y, x.numpy(), W)
    mod = QuantLinear(bits, gs, K, N, False)
    mod.qweight, mod.qzeros, mod.scales, mod.g_idx = layer.qweight, layer.qzeros, layer.scales, layer.g_idx
    mod = mod.to(DEV)
    _check_output(mod(x.to(DEV)), x.numpy(), W)
    assert mod._x_perm is not None


@pytest.mark.parametrize("bits", [3, 4])
def test_known_answer_integer_sums(bits):
    """w = arange % 4, x = ones, scale = 1, zero-point 1 (the reference's hand-run pattern,
    pycuda_warpper.py:330-343): every output is an exactly representable integer sum."""
    K, N = 1024, 256
    w = (np.arange(N * K, dtype=np.int64) % 4).reshape(N, K).astype(np.float32)
    qweight, qzeros, s16 = O.pack(w, np.ones((N, 1), np.float32), np.ones((N, 1), np.float32),
                                  np.zeros(K, np.int32), bits)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    x = torch.ones((1, K), dtype=torch.float16, device=DEV)
    y = ops.gemv(x, t(qweight), t(qzeros), t(s16), None, bits, -1)
    assert np.array_equal(y.cpu().numpy().astype(np.float64)[0], w.sum(axis=1))


def test_linearity_at_full_size():
    """Size-independent property on config 1: y(a + b) = y(a) + y(b) up to fp16 rounding of the outputs."""
    layer = synth.make_layer(3, 4096, 11008, 128, True, seed=5).to(DEV)
    mod = QuantLinear(3, 128, 4096, 11008, False)
    mod.qweight, mod.qzeros, mod.scales, mod.g_idx = layer.qweight, layer.qzeros, layer.scales, layer.g_idx
    mod = mod.to(DEV)
    a = (synth.make_x(1, 4096, seed=1) * 0.5).to(DEV)
    b = (synth.make_x(1, 4096, seed=2) * 0.5).to(DEV)
    ya, yb, yab = mod(a).float(), mod(b).float(), mod(a + b).float()
    # a + b is rounded to fp16 before the product; bound that separately
    scale = float(mod.scales.float().max()) * 8
    bound = 3 * 2.0 ** -11 * (ya.abs() + yb.abs() + yab.abs()) + 4096 ** 0.5 * 2.0 ** -11 * 4 * scale
    assert bool(((ya + yb - yab).abs() <= bound).all())


def test_error_reporting():
    layer = synth.make_layer(4, 256, 64, 128).to(DEV)
    x = synth.make_x(1, 256).to(DEV)
    with pytest.raises(RuntimeError):
        ops.gemv(x.cpu(), layer.qweight, layer.qzeros, layer.scales, layer.g_idx, 4, 128)
    with pytest.raises(ValueError):
        ops.gemv(x[:, :128].contiguous(), layer.qweight, layer.qzeros, layer.scales, layer.g_idx, 4, 128)
    with pytest.raises(ValueError):  # 9 rows is not a GEMV
        ops.gemv(synth.make_x(9, 256).to(DEV), layer.qweight, layer.qzeros, layer.scales, layer.g_idx, 4, 128)
    with pytest.raises(ValueError):  # 5 bits
        ops.gemv(x, layer.qweight, layer.qzeros, layer.scales, layer.g_idx, 5, 128)
    small = torch.zeros(16, dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError):
        ops.gemv(synth.make_x(1, 4096).to(DEV), *(lambda L: (L.qweight, L.qzeros, L.scales, L.g_idx))(
            synth.make_layer(4, 4096, 4096).to(DEV)), 4, 128, workspace=small)
    with pytest.raises(NotImplementedError):
        QuantLinear(5, 128, 256, 64, False)
    with pytest.raises(RuntimeError):
        QuantLinear(4, 128, 256, 64, False)(torch.zeros(1, 256))


@pytest.mark.parametrize("M", [1, 5, 48])
def test_traced_forward_equals_eager(M):
    """torch.compile(fullgraph=True) of a QuantLinear records the registered operator (no graph break, no ctypes
    call at trace time) and gives the eager result."""
    import torch._dynamo
    from autogptq.tvm_b200 import torch_ops  # noqa: F401
    bits, K, N, gs = 4, 512, 256, 128
    layer = synth.make_layer(bits, K, N, gs, True, bias=True, seed=3)
    mod = QuantLinear(bits, gs, K, N, True)
    mod.qweight, mod.qzeros, mod.scales, mod.g_idx, mod.bias = (layer.qweight, layer.qzeros, layer.scales,
                                                                  layer.g_idx, layer.bias)
    mod = mod.to(DEV)
    x = synth.make_x(M, K, seed=M, device=DEV)
    want = mod(x)                                   # eager: also builds the run-time layout
    torch._dynamo.reset()
    traced = torch.compile(mod, backend="eager", fullgraph=True)
    got = traced(x)
    assert torch.equal(got, want)
    y = torch.ops.b200gptq.quant_matmul(x, mod._qweight_run, mod.qzeros, mod.scales, mod._g_idx_run, mod._x_perm,
                                        mod.bias, bits, gs, mod._gemm_ok)
    assert torch.equal(y, want)


@pytest.mark.parametrize("bits,K,N,act_order", [(4, 11008, 4096, False), (3, 4096, 1056, False), (3, 4096, 1024, True),
                                                (4, 1024, 512, True)])
@pytest.mark.parametrize("M", [1, 4])
@pytest.mark.parametrize("kind", ["swiglu", "relu"])
def test_gemv_with_folded_activation(bits, K, N, act_order, M, kind):
    """b200gptq_gemv_ex / plan_create_ex: the activation applied inside the GEMV's read of x gives bit for bit what
    b200gptq_act followed by the plain GEMV gives (both fp16 paths and the integer path, with and without a gather)."""
    input_act = _lib.ACT_SWIGLU if kind == "swiglu" else _lib.ACT_RELU
    layer = synth.make_layer(bits, K, N, 128, act_order, bias=True, seed=K + N).to(DEV)
    if act_order:
        qw, perm, _ = ops.sort_rows(layer.qweight, layer.g_idx, bits)
    else:
        qw, perm = layer.qweight, None
    width = 2 * K if kind == "swiglu" else K
    u = synth.make_x(M, width, seed=M + 7, device=DEV)
    foldable = ops.can_fold_act(M, K, N, bits, 128, False, perm is not None, input_act)
    assert foldable == (not (kind == "swiglu" and act_order))
    if not foldable:
        with pytest.raises(ValueError):
            ops.gemv(u, qw, layer.qzeros, layer.scales, None, bits, 128, bias=layer.bias, x_perm=perm, input_act=input_act)
        return
    a = torch.empty((M, K), dtype=torch.float16, device=DEV)
    ops.act(u, a, K, kind == "swiglu")
    want = ops.gemv(a, qw, layer.qzeros, layer.scales, None, bits, 128, bias=layer.bias, x_perm=perm)
    got = ops.gemv(u, qw, layer.qzeros, layer.scales, None, bits, 128, bias=layer.bias, x_perm=perm, input_act=input_act)
    assert torch.equal(got, want)
    plan = ops.GemvPlan(qw, layer.qzeros, layer.scales, None, perm, layer.bias, M, bits, 128, None, input_act)
    assert torch.equal(plan.run(u), want)
    # the general kernel has no folded activation: asking for it is refused, not ignored
    with pytest.raises(ValueError):
        ops.gemv(u, layer.qweight, layer.qzeros, layer.scales, layer.g_idx, bits, 128, input_act=input_act)
