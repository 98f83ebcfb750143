"""ctypes binding of ``libb200gptq.so`` (the C ABI declared in ``include/b200gptq.h``).

There is no fallback: if the shared library is absent and cannot be built, importing
this module raises, and every operator of the package fails with it.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

OP_GEMV = 1
OP_GEMM = 2

_c_int = ctypes.c_int
_c_void_p = ctypes.c_void_p
_c_size_t = ctypes.c_size_t

_SIGNATURES = {
    "b200gptq_strerror": (ctypes.c_char_p, [_c_int]),
    "b200gptq_last_cuda_error": (_c_int, []),
    "b200gptq_abi_version": (_c_int, []),
    "b200gptq_dequant": (_c_int, [_c_void_p] * 4 + [_c_int] * 4 + [_c_void_p] * 3),
    "b200gptq_workspace_bytes": (_c_size_t, [_c_int] * 5),
    "b200gptq_workspace_status": (_c_int, [_c_void_p, _c_void_p, _c_void_p]),
    "b200gptq_gemv": (_c_int, [_c_void_p] * 8 + [_c_int] * 5 + [_c_void_p, _c_size_t, _c_void_p]),
    "b200gptq_gemv_tuned": (_c_int, [_c_void_p] * 8 + [_c_int] * 5 + [_c_void_p, _c_size_t, _c_int, _c_int, _c_void_p]),
    "b200gptq_gemv_ex": (_c_int, [_c_void_p] * 8 + [_c_int] * 5 + [_c_void_p, _c_size_t, _c_int, _c_int, _c_int, _c_void_p]),
    "b200gptq_gemv_plan_create": (_c_int, [_c_void_p] * 7 + [_c_int] * 7),
    "b200gptq_gemv_plan_create_ex": (_c_int, [_c_void_p] * 7 + [_c_int] * 8),
    "b200gptq_gemv_plan_run": (_c_int, [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_size_t, _c_void_p]),
    "b200gptq_gemv_plan_destroy": (None, [_c_void_p]),
    "b200gptq_gemv_path": (_c_int, [_c_int] * 6),
    "b200gptq_gemm_split": (_c_int, [_c_int] * 4 + [_c_void_p] * 2),
    "b200gptq_gemm": (_c_int, [_c_void_p] * 8 + [_c_int] * 5 + [_c_void_p, _c_size_t, _c_void_p]),
    "b200gptq_sort_rows": (_c_int, [_c_void_p] * 3 + [_c_int] * 3 + [_c_void_p] * 3),
    "b200gptq_pack_fields": (_c_int, [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p]),
    "b200gptq_tp_buffer_bytes": (_c_size_t, []),
    "b200gptq_gemv_tp": (_c_int, [_c_void_p] * 8 + [_c_int] * 5 + [_c_void_p, _c_size_t, _c_int, _c_int, _c_void_p,
                                  ctypes.c_longlong, _c_int, _c_int, _c_void_p]),
    "b200gptq_gemv_tp_ex": (_c_int, [_c_void_p] * 8 + [_c_int] * 5 + [_c_void_p, _c_size_t, _c_int, _c_int, _c_void_p,
                                     ctypes.c_longlong, _c_int, _c_int, _c_int, _c_void_p]),
    "b200gptq_tp_allreduce": (_c_int, [_c_void_p] * 2 + [_c_int] * 4 + [_c_void_p, ctypes.c_longlong, _c_void_p]),
    "b200gptq_tp_status": (_c_int, [_c_void_p, _c_void_p, _c_void_p]),
    "b200gptq_tp_enable_peer": (_c_int, [_c_int]),
    "b200gptq_tp_export": (_c_int, [_c_void_p, _c_void_p, _c_void_p]),
    "b200gptq_tp_open_peer": (_c_int, [_c_void_p, _c_void_p]),
    "b200gptq_tp_close_peer": (_c_int, [_c_void_p]),
    "b200gptq_tp_probe": (_c_int, [_c_void_p, _c_void_p]),
    "b200gptq_gemv_static": (_c_int, [_c_void_p] * 8 + [_c_int] * 5 + [_c_void_p]),
    "b200gptq_gemv_static_capacity": (_c_size_t, []),
    "b200gptq_gemv_static_status": (_c_int, [_c_void_p, _c_void_p]),
    "b200gptq_add_norm": (_c_int, [_c_void_p] * 5 + [_c_int, _c_int, ctypes.c_float, _c_int, _c_void_p]),
    "b200gptq_rope_cache": (_c_int, [_c_void_p] * 7 + [_c_int] * 5 + [_c_void_p]),
    "b200gptq_attn_decode": (_c_int, [_c_void_p] * 5 + [_c_int] * 4 + [ctypes.c_float, _c_void_p]),
    "b200gptq_attn_step": (_c_int, [_c_void_p] * 7 + [_c_int] * 5 + [ctypes.c_float, _c_void_p]),
    "b200gptq_act": (_c_int, [_c_void_p] * 2 + [_c_int] * 3 + [_c_void_p]),
    "b200gptq_dense_gemv": (_c_int, [_c_void_p] * 3 + [_c_int] * 3 + [_c_void_p]),
    "b200gptq_pick_local": (_c_int, [_c_void_p, _c_int, _c_int, _c_int, ctypes.c_longlong, _c_int, _c_int, _c_void_p,
                                     _c_void_p, ctypes.c_longlong, _c_void_p, _c_void_p]),
    "b200gptq_pick_final": (_c_int, [_c_void_p, _c_int, _c_int, _c_void_p, ctypes.c_longlong, _c_void_p, _c_void_p]),
}


def _load() -> ctypes.CDLL:
    path = _build.LIB_PATH
    if not os.path.isfile(path) or (_build.is_stale() and _build_possible()):
        if not _build_possible():
            raise ImportError(
                f"{path} is missing and nvcc is not available to build it; "
                "the B200 GPTQ kernels have no fallback implementation")
        _build.build()
    lib = ctypes.CDLL(path)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the library does not match the header
        fn.restype = res
        fn.argtypes = args
    return lib


def _build_possible() -> bool:
    import shutil
    return bool(shutil.which("nvcc")) or os.path.exists("/usr/local/cuda/bin/nvcc")


lib = _load()
LIB_PATH = _build.LIB_PATH


class B200GPTQError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib.b200gptq_strerror(status).decode()
        if status == -6:
            msg += f" (cudaError {lib.b200gptq_last_cuda_error()})"
        super().__init__(f"{where}: {msg} [status {status}]")


def check(status: int, where: str) -> None:
    if status != 0:
        if status in (-2, -3, -4):
            raise ValueError(str(B200GPTQError(status, where)))
        raise B200GPTQError(status, where)


PATH_STREAM = 1
PATH_GENERIC = 2
ACT_NONE, ACT_SWIGLU, ACT_RELU = 0, 1, 2


def gemv_path(M: int, K: int, N: int, bits: int, group_size: int, has_g_idx: bool) -> int:
    """Which kernel ``b200gptq_gemv`` runs: ``PATH_STREAM`` or ``PATH_GENERIC``."""
    return int(lib.b200gptq_gemv_path(M, K, N, bits, group_size, 1 if has_g_idx else 0))


def workspace_bytes(op: int, M: int, K: int, N: int, bits: int) -> int:
    return int(lib.b200gptq_workspace_bytes(op, M, K, N, bits))
