"""Functional wrappers: torch CUDA tensors in, C-ABI calls out.

Each function validates what the C side cannot see (device, dtype, contiguity),
passes raw device pointers plus the current CUDA stream, and raises on a non-zero
status.  Nothing here computes on the host.
"""
from __future__ import annotations

import sys
from typing import Optional, Tuple

import torch

from . import _lib

_workspaces = {}


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(name: str, t: torch.Tensor, dtype: torch.dtype) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: the B200 GPTQ kernels have no CPU path")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _stream(device: torch.device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(index)    # the handle without building a Stream object (2 us)


def get_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch shared by the calls issued on one device AND one stream.

    The kernels restore the scratch to its zero state, so one buffer serves every layer as long as calls are
    ordered on a stream; calls on different streams may overlap on the GPU and therefore get different buffers.
    A buffer that has to grow is replaced (its sticky status word travels to the new one).
    """
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, torch._C._cuda_getCurrentRawStream(index))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        size = max(nbytes, 1 << 20)
        new = torch.zeros(size, dtype=torch.uint8, device=device)
        if ws is not None:
            new[16380:16384].copy_(ws[16380:16384])
        ws = _workspaces[key] = new
    return ws


def check_status(device=None) -> None:
    """Raise if any kernel that used this module's scratch buffers on ``device`` gave up a bounded wait (its results
    were then undefined).  Synchronises the streams it looks at; meant for tests, benchmarks and the end of a run."""
    import ctypes
    for (index, stream), ws in list(_workspaces.items()):
        if device is not None and torch.device(device).index not in (None, index):
            continue
        word = ctypes.c_uint(0)
        with torch.cuda.device(index):
            _lib.check(_lib.lib.b200gptq_workspace_status(ws.data_ptr(), stream, ctypes.byref(word)),
                       "b200gptq_workspace_status")
        if word.value:
            raise RuntimeError(f"a kernel on cuda:{index} gave up a bounded wait (status word {word.value}): "
                               "results computed since the scratch was created are not trustworthy")


def layer_dims(qweight: torch.Tensor, bits: int) -> Tuple[int, int]:
    return qweight.shape[0] * 32 // bits, qweight.shape[1]


def dequantize(qweight, qzeros, scales, g_idx, bits: int, group_size: int,
               want_q: bool = True, want_w: bool = True):
    """Return ``(q int8 [K,N] | None, W fp16 [K,N] | None)`` computed on the GPU."""
    _need_cuda("qweight", qweight, torch.int32)
    _need_cuda("qzeros", qzeros, torch.int32)
    _need_cuda("scales", scales, torch.float16)
    if g_idx is not None:
        _need_cuda("g_idx", g_idx, torch.int32)
    K, N = layer_dims(qweight, bits)
    dev = qweight.device
    q = torch.empty((K, N), dtype=torch.int8, device=dev) if want_q else None
    w = torch.empty((K, N), dtype=torch.float16, device=dev) if want_w else None
    with torch.cuda.device(dev):
        st = _lib.lib.b200gptq_dequant(_ptr(qweight), _ptr(qzeros), _ptr(scales), _ptr(g_idx), K, N, bits,
                                       group_size, _ptr(q), _ptr(w), _stream(dev))
    _lib.check(st, "b200gptq_dequant")
    return q, w


def pack_fields(vals, bits: int):
    """Pack ``vals`` (int32 CUDA tensor ``[R, C]``, ``R % 32 == 0``) along dim 0 into GPTQ int32 words
    ``[R/32*bits, C]``; values wider than ``bits`` spill into neighbouring fields like the reference's pack."""
    _need_cuda("vals", vals, torch.int32)
    if vals.dim() != 2 or vals.shape[0] % 32 != 0:
        raise ValueError(f"vals must be [R, C] with R % 32 == 0, got {tuple(vals.shape)}")
    R, C = vals.shape
    out = torch.empty((R // 32 * bits, C), dtype=torch.int32, device=vals.device)
    with torch.cuda.device(vals.device):
        st = _lib.lib.b200gptq_pack_fields(_ptr(vals), R, C, bits, _ptr(out), _stream(vals.device))
    _lib.check(st, "b200gptq_pack_fields")
    return out


def sort_rows(qweight, g_idx, bits: int):
    """Re-order the rows of an act-order layer by group.  Returns
    ``(qweight_sorted, perm, g_idx_sorted)``; ``perm`` is the stable argsort of ``g_idx``."""
    _need_cuda("qweight", qweight, torch.int32)
    _need_cuda("g_idx", g_idx, torch.int32)
    K, N = layer_dims(qweight, bits)
    perm = torch.sort(g_idx.to(torch.int64), stable=True).indices.to(torch.int32).contiguous()
    out = torch.empty_like(qweight)
    g_sorted = torch.empty_like(g_idx)
    dev = qweight.device
    with torch.cuda.device(dev):
        st = _lib.lib.b200gptq_sort_rows(_ptr(qweight), _ptr(g_idx), _ptr(perm), K, N, bits, _ptr(out),
                                         _ptr(g_sorted), _stream(dev))
    _lib.check(st, "b200gptq_sort_rows")
    return out, perm, g_sorted


def _matmul(fn_name: str, op: int, x, qweight, qzeros, scales, g_idx, x_perm, bias, bits, group_size,
            out, workspace, tuning=None, input_act: int = 0):
    _need_cuda("x", x, torch.float16)
    _need_cuda("qweight", qweight, torch.int32)
    _need_cuda("qzeros", qzeros, torch.int32)
    _need_cuda("scales", scales, torch.float16)
    if g_idx is not None:
        _need_cuda("g_idx", g_idx, torch.int32)
    if x_perm is not None:
        _need_cuda("x_perm", x_perm, torch.int32)
    if bias is not None:
        _need_cuda("bias", bias, torch.float16)
    K, N = layer_dims(qweight, bits)
    xk = 2 * K if input_act == _lib.ACT_SWIGLU else K
    if x.dim() != 2 or x.shape[1] != xk:
        raise ValueError(f"x must be [M, {xk}], got {tuple(x.shape)}")
    M = x.shape[0]
    dev = x.device
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=dev)
    else:
        _need_cuda("out", out, torch.float16)
        if tuple(out.shape) != (M, N):
            raise ValueError(f"out must be [{M}, {N}]")
    need = _lib.workspace_bytes(op, M, K, N, bits)
    if workspace is None:
        workspace = get_workspace(dev, need)
    with torch.cuda.device(dev):
        if tuning is not None or input_act:
            fn_name = "b200gptq_gemv_ex"
            st = _lib.lib.b200gptq_gemv_ex(_ptr(x), _ptr(qweight), _ptr(qzeros), _ptr(scales), _ptr(g_idx),
                                           _ptr(x_perm), _ptr(bias), _ptr(out), M, K, N, bits, group_size,
                                           _ptr(workspace), workspace.numel() * workspace.element_size(),
                                           int(tuning[0]) if tuning else 0, int(tuning[1]) if tuning else 0,
                                           int(input_act), _stream(dev))
        else:
            st = getattr(_lib.lib, fn_name)(_ptr(x), _ptr(qweight), _ptr(qzeros), _ptr(scales), _ptr(g_idx),
                                            _ptr(x_perm), _ptr(bias), _ptr(out), M, K, N, bits, group_size,
                                            _ptr(workspace), workspace.numel() * workspace.element_size(),
                                            _stream(dev))
    _lib.check(st, fn_name)
    return out


def gemv(x, qweight, qzeros, scales, g_idx, bits: int, group_size: int, bias=None, x_perm=None,
         out=None, workspace=None, tuning=None, input_act: int = 0):
    """Decode GEMV, ``x`` fp16 ``[M<=8, K]`` -> fp16 ``[M, N]``.  ``tuning = (slices_per_sm, ctas_per_sm)`` and
    ``input_act`` (``_lib.ACT_SWIGLU``: ``x`` is ``[M, 2K] = [gate | up]``; ``_lib.ACT_RELU``) select
    ``b200gptq_gemv_ex`` (see the header); the defaults mean the plain call.  Raises when the activation cannot be
    folded for this layer (see :func:`can_fold_act`)."""
    return _matmul("b200gptq_gemv", _lib.OP_GEMV, x, qweight, qzeros, scales, g_idx, x_perm, bias, bits,
                   group_size, out, workspace, tuning, input_act)


def can_fold_act(M: int, K: int, N: int, bits: int, group_size: int, has_g_idx: bool, has_perm: bool, input_act: int) -> bool:
    """Whether ``b200gptq_gemv_ex`` folds ``input_act`` into this GEMV (only the streaming kernel does, and SwiGLU not
    together with a gather); otherwise the caller runs :func:`act` first."""
    if not input_act:
        return True
    if _lib.gemv_path(M, K, N, bits, group_size, has_g_idx) != _lib.PATH_STREAM:
        return False
    return not (input_act == _lib.ACT_SWIGLU and has_perm)


def gemm(x, qweight, qzeros, scales, g_idx, bits: int, group_size: int, bias=None, x_perm=None,
         out=None, workspace=None):
    """Prefill dequant-GEMM on tcgen05, ``x`` fp16 ``[M, K]`` -> fp16 ``[M, N]``."""
    return _matmul("b200gptq_gemm", _lib.OP_GEMM, x, qweight, qzeros, scales, g_idx, x_perm, bias, bits,
                   group_size, out, workspace)


class GemvPlan:
    """A prepared decode GEMV for one layer and one row count (``b200gptq_gemv_plan_*``): kernel choice, work split
    and TMA descriptors are built once, a call is one kernel launch.  Keeps the layer's tensors alive."""

    def __init__(self, qweight, qzeros, scales, g_idx, x_perm, bias, M: int, bits: int, group_size: int, tuning=None,
                 input_act: int = 0):
        _need_cuda("qweight", qweight, torch.int32)
        _need_cuda("qzeros", qzeros, torch.int32)
        _need_cuda("scales", scales, torch.float16)
        for name, t, dt in (("g_idx", g_idx, torch.int32), ("x_perm", x_perm, torch.int32), ("bias", bias, torch.float16)):
            if t is not None:
                _need_cuda(name, t, dt)
        self._keep = (qweight, qzeros, scales, g_idx, x_perm, bias)
        self.M = M
        self.K, self.N = layer_dims(qweight, bits)
        self.device = qweight.device
        import ctypes
        handle = ctypes.c_void_p(0)
        self.xk = 2 * self.K if input_act == _lib.ACT_SWIGLU else self.K
        st = _lib.lib.b200gptq_gemv_plan_create_ex(ctypes.byref(handle), _ptr(qweight), _ptr(qzeros), _ptr(scales),
                                                   _ptr(g_idx), _ptr(x_perm), _ptr(bias), M, self.K, self.N, bits,
                                                   group_size, int(tuning[0]) if tuning else 0,
                                                   int(tuning[1]) if tuning else 0, int(input_act))
        _lib.check(st, "b200gptq_gemv_plan_create_ex")
        self._handle = handle
        self._need = _lib.workspace_bytes(_lib.OP_GEMV, M, self.K, self.N, bits)
        self._index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._run = _lib.lib.b200gptq_gemv_plan_run

    def run(self, x, out=None):
        if not x.is_cuda or x.dtype != torch.float16 or not x.is_contiguous() or tuple(x.shape) != (self.M, self.xk):
            raise ValueError(f"x must be a contiguous fp16 CUDA tensor [{self.M}, {self.xk}]")
        if out is None:
            out = torch.empty((self.M, self.N), dtype=torch.float16, device=x.device)
        ws = get_workspace(x.device, self._need)      # one buffer per (device, stream)
        st = _lib.lib.b200gptq_gemv_plan_run(self._handle, x.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(),
                                             torch.cuda.current_stream(x.device).cuda_stream)
        if st:
            _lib.check(st, "b200gptq_gemv_plan_run")
        return out

    def launch(self, x, out_shape):
        """:meth:`run` for a caller that has already checked ``x`` (contiguous fp16 on this plan's device, the plan's
        row count): allocates ``out`` with ``out_shape`` and launches.  The host side of a decode GEMV is most of its
        end-to-end time (25 us against 8 us on the device before this path existed), so nothing here builds a Stream
        or a device-guard object unless the current device is another one."""
        index = self._index
        out = torch.empty(out_shape, dtype=torch.float16, device=self.device)
        if torch._C._cuda_getDevice() != index:
            with torch.cuda.device(index):
                return self.run(x, out=out.view(self.M, self.N)).view(out_shape)
        stream = torch._C._cuda_getCurrentRawStream(index)
        ws = _workspaces.get((index, stream))
        if ws is None or ws.numel() < self._need:
            ws = get_workspace(self.device, self._need)
        st = self._run(self._handle, x.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), stream)
        if st:
            _lib.check(st, "b200gptq_gemv_plan_run")
        return out

    def __del__(self, _finalizing=sys.is_finalizing):
        h, self._handle = getattr(self, "_handle", None), None
        if h and not _finalizing():     # at interpreter exit the host object is reclaimed with the process
            _lib.lib.b200gptq_gemv_plan_destroy(h)


def gemv_tp(x, qweight, qzeros, scales, g_idx, bits: int, group_size: int, exchange, bias=None, x_perm=None,
            out=None, workspace=None, tuning=None, input_act: int = 0):
    """Row-parallel decode GEMV with the sum over ranks fused in (``b200gptq_gemv_tp``): ``x`` is this rank's slice of
    the input ``[M<=8, K_local]``, the packed buffers are this rank's shard, ``bias`` is the full bias (the same on
    every rank).  ``exchange`` is a :class:`exchange.PeerExchange`.  Returns the complete result on every rank."""
    _need_cuda("x", x, torch.float16)
    _need_cuda("qweight", qweight, torch.int32)
    _need_cuda("qzeros", qzeros, torch.int32)
    _need_cuda("scales", scales, torch.float16)
    for name, t, dt in (("g_idx", g_idx, torch.int32), ("x_perm", x_perm, torch.int32), ("bias", bias, torch.float16)):
        if t is not None:
            _need_cuda(name, t, dt)
    K, N = layer_dims(qweight, bits)
    xk = 2 * K if input_act == _lib.ACT_SWIGLU else K
    if x.dim() != 2 or x.shape[1] != xk:
        raise ValueError(f"x must be [M, {xk}], got {tuple(x.shape)}")
    M = x.shape[0]
    dev = x.device
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=dev)
    if workspace is None:
        workspace = get_workspace(dev, _lib.workspace_bytes(_lib.OP_GEMV, M, K, N, bits))
    with torch.cuda.device(dev):
        st = _lib.lib.b200gptq_gemv_tp_ex(_ptr(x), _ptr(qweight), _ptr(qzeros), _ptr(scales), _ptr(g_idx), _ptr(x_perm),
                                          _ptr(bias), _ptr(out), M, K, N, bits, group_size, _ptr(workspace),
                                          workspace.numel() * workspace.element_size(), exchange.rank, exchange.world,
                                          exchange.peer_table, exchange.timeout_cycles,
                                          int(tuning[0]) if tuning else 0, int(tuning[1]) if tuning else 0,
                                          int(input_act), _stream(dev))
    _lib.check(st, "b200gptq_gemv_tp_ex")
    return out


def tp_allreduce(y, exchange, bias=None):
    """In place ``y[M<=8, N] = sum over ranks of y (+ bias)`` through the peer-memory exchange."""
    _need_cuda("y", y, torch.float16)
    M, N = y.shape
    with torch.cuda.device(y.device):
        st = _lib.lib.b200gptq_tp_allreduce(_ptr(y), _ptr(bias), M, N, exchange.rank, exchange.world,
                                            exchange.peer_table, exchange.timeout_cycles, _stream(y.device))
    _lib.check(st, "b200gptq_tp_allreduce")
    return y


def gemv_static(x, qweight, qzeros, scales, g_idx, bits: int, group_size: int, bias=None, x_perm=None, out=None):
    """Decode GEMV through ``b200gptq_gemv_static``: same results as :func:`gemv`, but the kernels'
    scratch is the fixed array inside the library, so nothing is allocated for the call except (when
    ``out`` is not given) the result tensor.  Meant for hosts that cannot allocate device memory at
    launch time; calls on one device must be ordered on a stream because they share that array."""
    _need_cuda("x", x, torch.float16)
    _need_cuda("qweight", qweight, torch.int32)
    _need_cuda("qzeros", qzeros, torch.int32)
    _need_cuda("scales", scales, torch.float16)
    for name, t, dt in (("g_idx", g_idx, torch.int32), ("x_perm", x_perm, torch.int32), ("bias", bias, torch.float16)):
        if t is not None:
            _need_cuda(name, t, dt)
    K, N = layer_dims(qweight, bits)
    if x.dim() != 2 or x.shape[1] != K:
        raise ValueError(f"x must be [M, {K}], got {tuple(x.shape)}")
    M = x.shape[0]
    dev = x.device
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        st = _lib.lib.b200gptq_gemv_static(_ptr(x), _ptr(qweight), _ptr(qzeros), _ptr(scales), _ptr(g_idx),
                                           _ptr(x_perm), _ptr(bias), _ptr(out), M, K, N, bits, group_size,
                                           _stream(dev))
    _lib.check(st, "b200gptq_gemv_static")
    return out


# ---- decode-step helpers (see include/b200gptq.h) -----------------------------------------------
def add_norm(x, add, w, beta, out, eps: float, rms: bool):
    """In place ``x += add`` (if given), then ``out = norm(x) * w (+ beta)``; x, out fp16 ``[rows, H]``."""
    rows, H = x.shape
    with torch.cuda.device(x.device):
        st = _lib.lib.b200gptq_add_norm(_ptr(x), _ptr(add), _ptr(w), _ptr(beta), _ptr(out), rows, H, eps,
                                        1 if rms else 0, _stream(x.device))
    _lib.check(st, "b200gptq_add_norm")
    return out


def rope_cache(qkv, cos, sin, pos, q_out, k_cache, v_cache, heads: int, hd: int, rope: bool):
    B, max_seq = k_cache.shape[0], k_cache.shape[2]
    with torch.cuda.device(qkv.device):
        st = _lib.lib.b200gptq_rope_cache(_ptr(qkv), _ptr(cos), _ptr(sin), _ptr(pos), _ptr(q_out), _ptr(k_cache),
                                          _ptr(v_cache), B, heads, hd, max_seq, 1 if rope else 0, _stream(qkv.device))
    _lib.check(st, "b200gptq_rope_cache")
    return q_out


def attn_decode(q, k_cache, v_cache, pos, out, heads: int, hd: int):
    B, max_seq = k_cache.shape[0], k_cache.shape[2]
    with torch.cuda.device(q.device):
        st = _lib.lib.b200gptq_attn_decode(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(pos), _ptr(out), B, heads, hd,
                                           max_seq, 1.0 / (hd ** 0.5), _stream(q.device))
    _lib.check(st, "b200gptq_attn_decode")
    return out


def gemm_split(M: int, K: int, N: int, bits: int):
    """``b200gptq_gemm_split``: (thread blocks that share one tile's K, thread blocks per SM) of :func:`gemm` for this
    problem on the current device.  Host-only."""
    import ctypes
    sp, per = ctypes.c_int(0), ctypes.c_int(0)
    _lib.check(_lib.lib.b200gptq_gemm_split(M, K, N, bits, ctypes.byref(sp), ctypes.byref(per)), "b200gptq_gemm_split")
    return sp.value, per.value


def pick_local(logits, valid: int, base_index: int, world: int, rank: int, slots, tokens, max_token: int, pos_inc=None):
    """``b200gptq_pick_local``: greedy pick over this rank's fp16 ``logits[rows, ld]`` (columns ``[0, valid)``)."""
    _need_cuda("logits", logits, torch.float16)
    rows, ld = logits.shape
    with torch.cuda.device(logits.device):
        st = _lib.lib.b200gptq_pick_local(_ptr(logits), rows, ld, valid, base_index, world, rank, _ptr(slots),
                                          _ptr(tokens), max_token, _ptr(pos_inc), _stream(logits.device))
    _lib.check(st, "b200gptq_pick_local")


def pick_final(slots, world: int, tokens, max_token: int, pos_inc=None):
    """``b200gptq_pick_final``: the winning rank's token per row from the summed ``slots[rows, 4 * world]``."""
    _need_cuda("slots", slots, torch.float16)
    with torch.cuda.device(slots.device):
        st = _lib.lib.b200gptq_pick_final(_ptr(slots), slots.shape[0], world, _ptr(tokens), max_token, _ptr(pos_inc),
                                          _stream(slots.device))
    _lib.check(st, "b200gptq_pick_final")


def attn_step(qkv, cos_t, sin_t, pos, k_cache, v_cache, out, heads: int, hd: int, rope: bool):
    """:func:`rope_cache` and :func:`attn_decode` as one launch (``b200gptq_attn_step``): ``qkv`` ``[B, 3*heads*hd]`` of
    the new token in, attention output ``[B, heads*hd]`` out, caches updated at position ``pos[0]``."""
    B, max_seq = k_cache.shape[0], k_cache.shape[2]
    with torch.cuda.device(qkv.device):
        st = _lib.lib.b200gptq_attn_step(_ptr(qkv), _ptr(cos_t), _ptr(sin_t), _ptr(pos), _ptr(k_cache), _ptr(v_cache),
                                         _ptr(out), B, heads, hd, max_seq, 1 if rope else 0, 1.0 / (hd ** 0.5),
                                         _stream(qkv.device))
    _lib.check(st, "b200gptq_attn_step")
    return out


def act(u, out, inter: int, gated: bool):
    with torch.cuda.device(u.device):
        st = _lib.lib.b200gptq_act(_ptr(u), _ptr(out), u.shape[0], inter, 1 if gated else 0, _stream(u.device))
    _lib.check(st, "b200gptq_act")
    return out


def dense_gemv(x, w, out=None):
    """``y = x @ w.T`` for up to 8 rows of ``x`` (fp16 ``[M, K]``) and a dense fp16 ``w`` ``[N, K]``: the vocabulary
    projection of a decode step as one pass over ``w`` (``b200gptq_dense_gemv``)."""
    _need_cuda("x", x, torch.float16)
    _need_cuda("w", w, torch.float16)
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1] or not 1 <= x.shape[0] <= 8:
        raise ValueError("dense_gemv: x [M <= 8, K] and w [N, K] expected")
    if out is None:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float16, device=x.device)
    with torch.cuda.device(x.device):
        st = _lib.lib.b200gptq_dense_gemv(_ptr(x), _ptr(w), _ptr(out), x.shape[0], x.shape[1], w.shape[0], _stream(x.device))
    _lib.check(st, "b200gptq_dense_gemv")
    return out
