"""Host-side dispatch of QuantLinear.forward (no GPU): which entry point a given number of rows
reaches.  The reference dispatches on M in TVMHandler.__call__ (tvm_untils/pycuda_warpper.py:138-189:
m == 1 -> GEMV kernel, otherwise the padded GEMM buckets); here M <= 8 goes to the GEMV, more rows to
the tensor-core GEMM for 3/4-bit layers and to GEMV passes of 8 rows for 2/8-bit layers."""
import pytest
import torch

from autogptq.tvm_b200 import qlinear as ql


class _FakeCuda(torch.Tensor):
    """A CPU tensor that claims to live on a GPU, so that forward() gets as far as its dispatch."""
    is_cuda = property(lambda self: True)


def _layer(bits, groupsize=128):
    m = ql.QuantLinear(bits, groupsize, 256, 64, False)
    m._ready = lambda: True
    m._qweight_run, m._g_idx_run, m._x_perm = m.qweight, None, None
    m._gemm_ok = bits in (3, 4) and groupsize % 32 == 0
    return m


@pytest.mark.parametrize("bits,M,want", [
    (4, 1, ["gemv:1"]), (4, 8, ["gemv:8"]), (4, 9, ["gemm:9"]), (3, 16, ["gemm:16"]), (4, 2048, ["gemm:2048"]),
    (8, 8, ["gemv:8"]), (8, 20, ["gemv:8", "gemv:8", "gemv:4"]), (2, 9, ["gemv:8", "gemv:1"]),
    # a group size that cuts through 32-row blocks cannot use the tensor-core kernel (one group per block)
    ((4, 16), 16, ["gemv:8", "gemv:8"]),
])
def test_rows_decide_the_entry_point(monkeypatch, bits, M, want):
    groupsize = 128
    if isinstance(bits, tuple):
        bits, groupsize = bits
    calls = []

    def fake(name):
        def f(x, *args, out=None, **kw):
            calls.append(f"{name}:{x.shape[0]}")
            return out if out is not None else torch.zeros((x.shape[0], 64), dtype=torch.float16)
        return f

    class FakePlan:   # up to 8 rows go through a prepared launch (ops.GemvPlan)
        def __init__(self, *a, **k):
            self._keep = (None,) * 6

        def run(self, x, out=None):
            return fake("gemv")(x, out=out)

    monkeypatch.setattr(ql.ops, "GemvPlan", FakePlan)
    monkeypatch.setattr(ql.ops, "gemv", fake("gemv"))
    monkeypatch.setattr(ql.ops, "gemm", fake("gemm"))
    monkeypatch.setattr(torch.cuda, "device", lambda d: __import__("contextlib").nullcontext())
    monkeypatch.setattr(torch, "empty", lambda *a, device=None, **k: torch.zeros(*a, **k))
    x = torch.zeros((M, 256), dtype=torch.float16).as_subclass(_FakeCuda)
    y = _layer(bits, groupsize).forward(x)
    assert calls == want
    assert tuple(y.shape) == (M, 64)


def test_decode_positions_are_checked_on_the_host():
    from autogptq.tvm_b200.decoder import check_positions
    check_positions(512, 256, 768)
    with pytest.raises(ValueError):
        check_positions(512, 257, 768)
    with pytest.raises(ValueError):
        check_positions(-1, 1, 768)


def test_registered_operator_has_a_shape_rule():
    """torch.ops.b200gptq.quant_matmul is registered with a fake (meta) implementation: tracing tools can infer the
    output of a QuantLinear without running it (the reference module is not traceable at all: it calls pycuda)."""
    import torch
    from autogptq.tvm_b200 import torch_ops  # noqa: F401  (registers the operator)
    op = torch.ops.b200gptq.quant_matmul
    K, N, bits = 256, 96, 4
    x = torch.empty((5, K), dtype=torch.float16, device="meta")
    qweight = torch.empty((K // 32 * bits, N), dtype=torch.int32, device="meta")
    qzeros = torch.empty((2, N // 32 * bits), dtype=torch.int32, device="meta")
    scales = torch.empty((2, N), dtype=torch.float16, device="meta")
    y = op(x, qweight, qzeros, scales, None, None, None, bits, 128, True)
    assert y.shape == (5, N) and y.dtype == torch.float16 and y.device.type == "meta"
    import pytest
    with pytest.raises(Exception):
        op(torch.empty((5, K + 32), dtype=torch.float16, device="meta"), qweight, qzeros, scales, None, None, None,
           bits, 128, True)


def test_gemm_work_split_rule():
    """b200gptq_gemm_split is host-only (without a device it plans for 148 SMs): K is split only for up to 128 rows
    and while every run keeps 16 k-tiles (40 above 64 rows); the second CTA per SM comes only for up to 64 rows and
    only where it shortens waves x k-tiles."""
    from autogptq.tvm_b200 import ops
    assert ops.gemm_split(16, 4096, 4096, 4) == (4, 1)        # 32 column tiles on 148 SMs: four runs of 16 k-tiles
    assert ops.gemm_split(128, 4096, 4096, 4) == (1, 1)       # 32 k-tiles per run would be too few above 64 rows
    assert ops.gemm_split(128, 11008, 4096, 4) == (4, 1)      # 172 k-tiles: four runs of 43
    assert ops.gemm_split(16, 4096, 12288, 4) == (3, 2)       # 96 tiles: three runs, two CTAs per SM
    assert ops.gemm_split(64, 9216, 27648, 3) == (1, 2)       # 216 tiles: one wave of two per SM instead of two waves
    assert ops.gemm_split(16, 9216, 9216, 3)[0] > 1
    assert ops.gemm_split(256, 4096, 4096, 4) == (1, 1)       # more than one row tile: never split
    assert ops.gemm_split(2048, 4096, 12288, 4) == (1, 1)
    with pytest.raises(ValueError):
        ops.gemm_split(16, 4095, 4096, 4)
