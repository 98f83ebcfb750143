"""Exchange buffers for the fused tensor-parallel all-reduce (``b200gptq_gemv_tp`` / ``b200gptq_tp_allreduce``).

Every rank of a single-node process group allocates one buffer, exports its CUDA IPC handle, and maps the other
ranks' buffers into its OWN device's address space (``b200gptq_tp_open_peer``: ``cudaIpcOpenMemHandle`` with this
rank's device current, which also enables peer access), after which this rank's kernels can store into any
rank's buffer.  PyTorch is plumbing here: it owns the memory and carries the handles over the process group; the
exchange itself is done by the library's kernels.
"""
from __future__ import annotations

import sys

import ctypes
from typing import List

import torch
import torch.distributed as dist

from . import _lib


class PeerExchange:
    """The exchange buffers of all ranks of ``group`` as seen from this rank."""

    def __init__(self, device: torch.device, group=None, timeout_cycles: int = 0):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("PeerExchange needs an initialised process group")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("the fused all-reduce serves up to 8 ranks of one node")
        self.device = torch.device(device)
        self.timeout_cycles = int(timeout_cycles)
        nbytes = int(_lib.lib.b200gptq_tp_buffer_bytes())
        self.own = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)   # zero-filled once
        torch.cuda.synchronize(self.device)
        # the IPC handle names the allocation the buffer was carved from; the buffer starts `offset` bytes into it
        hbuf = ctypes.create_string_buffer(64)
        off = ctypes.c_size_t(0)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib.b200gptq_tp_export(self.own.data_ptr(), hbuf, ctypes.byref(off)), "b200gptq_tp_export")
        handle, offset = hbuf.raw, int(off.value)
        gathered: List[object] = [None] * self.world
        dist.all_gather_object(gathered, (handle, offset, self.device.index), group=group)
        self._mapped: List[int] = []
        ptrs: List[int] = []
        with torch.cuda.device(self.device):
            for r, (h, off, peer_dev) in enumerate(gathered):
                if r == self.rank:
                    ptrs.append(self.own.data_ptr())
                    continue
                if not torch.cuda.can_device_access_peer(self.device.index, peer_dev):
                    raise RuntimeError(f"GPU {self.device.index} cannot address GPU {peer_dev}: no fused all-reduce")
                base = ctypes.c_void_p(0)
                buf = ctypes.create_string_buffer(h, len(h))
                _lib.check(_lib.lib.b200gptq_tp_open_peer(buf, ctypes.byref(base)), "b200gptq_tp_open_peer")
                self._mapped.append(base.value)
                ptrs.append(base.value + off)
            # every mapping must be readable (and hold the zeros its owner wrote) before any kernel touches it
            for r, p in enumerate(ptrs):
                word = ctypes.c_uint(1)
                _lib.check(_lib.lib.b200gptq_tp_probe(p, ctypes.byref(word)), "b200gptq_tp_probe")
                if word.value != 0:
                    raise RuntimeError(f"exchange buffer of rank {r} is not zero-filled as seen from rank {self.rank}")
        self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        dist.barrier(group=group)               # nobody stores into a buffer before everybody has mapped and checked

    @property
    def peer_table(self):
        """Host array of the ``world`` device pointers, as the C ABI wants it."""
        return self._ptrs

    def status(self) -> int:
        """The sticky status word of this rank's buffer (0: every wait was satisfied); synchronises the stream."""
        out = ctypes.c_uint(0)
        with torch.cuda.device(self.device):
            st = _lib.lib.b200gptq_tp_status(self.own.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream,
                                             ctypes.byref(out))
        _lib.check(st, "b200gptq_tp_status")
        return int(out.value)

    def clear_status(self) -> None:
        self.own[:4].zero_()

    def close(self) -> None:
        """Unmap the peers' buffers.  Collective in spirit: call it on every rank once no kernel that uses the
        buffers is in flight anywhere (a barrier after the last synchronise), and before the owners free them."""
        mapped, self._mapped = self._mapped, []
        if mapped:
            torch.cuda.synchronize(self.device)
            with torch.cuda.device(self.device):
                for base in mapped:
                    _lib.lib.b200gptq_tp_close_peer(base)

    def __del__(self, _finalizing=sys.is_finalizing):
        if not _finalizing():
            try:
                self.close()
            except Exception:
                pass
