"""b200gptq_gemv_static: the GEMV entry point whose scratch is built into the library.

It serves hosts that cannot allocate device memory when they launch (a plugin inside another
runtime's callback, an engine with a frozen memory plan).  The kernels are the ones behind
b200gptq_gemv, so the results must be the same; what is tested here is the scratch handling: the
built-in array is found on first use, is shared by consecutive calls of different shapes without
any clearing by the caller, and oversized problems are refused instead of overrunning it.

This file sorts last on purpose: a run that stops at the first failure has then already executed
every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from autogptq.tvm_b200 import _lib, ops, synth
    DEV = torch.device("cuda:0")


CALLS = [
    # bits, K, N, group_size, act_order (g_idx passed), M, bias
    (3, 4096, 11008, 128, False, 1, False),   # streaming kernel, K split across CTAs
    (4, 4096, 4096, 128, False, 4, True),     # streaming kernel, another shape right after
    (4, 2048, 1056, 64, True, 3, False),      # general kernel (explicit g_idx), K split as well
    (3, 4096, 11008, 128, False, 8, False),   # back to the first shape with more rows
]


def test_two_and_more_calls_in_a_row_match_the_caller_scratch_entry_point():
    outs = []
    for bits, K, N, gs, act, M, bias in CALLS:
        layer = synth.make_layer(bits, K, N, gs, act, bias=bias, seed=K + N + M, device=DEV)
        x = synth.make_x(M, K, seed=M, device=DEV)
        g = layer.g_idx if act else None
        want = ops.gemv(x, layer.qweight, layer.qzeros, layer.scales, g, bits, gs, bias=layer.bias)
        got = ops.gemv_static(x, layer.qweight, layer.qzeros, layer.scales, g, bits, gs, bias=layer.bias)
        again = ops.gemv_static(x, layer.qweight, layer.qzeros, layer.scales, g, bits, gs, bias=layer.bias)
        outs.append((want, got, again))
    torch.cuda.synchronize()
    for want, got, again in outs:
        # same kernels, fixed summation order: equal bit for bit, which is inside every tolerance used elsewhere
        assert torch.equal(got, want)
        assert torch.equal(again, want)
        assert bool(torch.isfinite(got.float()).all())


def test_first_use_on_a_side_stream():
    """The entry point does no clearing of its own (its array is zero-initialised storage), so a call on a
    non-default, non-blocking stream needs no ordering against the default stream."""
    layer = synth.make_layer(4, 2048, 1056, 64, True, seed=9, device=DEV)      # general kernel: counters + partial sums
    x = synth.make_x(2, 2048, seed=9, device=DEV)
    want = ops.gemv(x, layer.qweight, layer.qzeros, layer.scales, layer.g_idx, 4, 64)
    torch.cuda.synchronize()
    side = torch.cuda.Stream(DEV)
    with torch.cuda.stream(side):
        got = ops.gemv_static(x, layer.qweight, layer.qzeros, layer.scales, layer.g_idx, 4, 64)
    side.synchronize()
    assert torch.equal(got, want)


def test_capacity_is_enforced():
    cap = int(_lib.lib.b200gptq_gemv_static_capacity())
    assert cap == 4 << 20
    bits, K, N, M = 8, 256, 262144, 8   # 8-bit layers take the general kernel, whose partial sums need M*N floats
    assert _lib.workspace_bytes(_lib.OP_GEMV, M, K, N, bits) > cap
    layer = synth.make_layer(bits, K, N, 128, False, seed=1, device=DEV)
    x = synth.make_x(M, K, seed=1, device=DEV)
    with pytest.raises(RuntimeError, match="capacity"):
        ops.gemv_static(x, layer.qweight, layer.qzeros, layer.scales, None, bits, 128)
    # the same problem still runs with caller-provided scratch
    y = ops.gemv(x, layer.qweight, layer.qzeros, layer.scales, None, bits, 128)
    assert bool(torch.isfinite(y.float()).all())


def test_status_of_the_built_in_scratch_is_clear():
    """b200gptq_gemv_static_status: no bounded wait of a kernel that used the built-in scratch has run out."""
    import ctypes
    word = ctypes.c_uint(7)
    with torch.cuda.device(0):
        st = _lib.lib.b200gptq_gemv_static_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(word))
    assert st == 0 and word.value == 0
