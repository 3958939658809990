"""Peer-mapped buffers for the tensor-parallel all-reduce kernel (q40_tp_* in include/q40b200.h).

One process per GPU.  `PeerBuffers` allocates this rank's buffer through the library (a plain device
allocation with a CUDA IPC handle), exchanges the handles over the process group's host channel and maps
the other ranks' buffers.  `allreduce_norm` enqueues the fused all-reduce + residual add + RMSNorm launch
that replaces `dist.all_reduce` after wo and w2 (hf_model_q40_kv_shared.py:258-261).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ._lib import Q40Error, check, lib


def layout(world: int, max_rows: int, dim: int):
    """(offset of the receive areas, total bytes) of a rank's buffer; a receive area is
    [2 slots][world][max_rows][dim / 4] lines of four 32-bit words {2 fp16, flag, 2 fp16, flag}."""
    out = (ctypes.c_size_t * 2)()
    check(lib.q40_tp_layout(world, max_rows, dim, out), "q40_tp_layout")
    return int(out[0]), int(out[1])


class RawBuffer:
    """A device allocation made by the library, visible to torch through __cuda_array_interface__."""

    def __init__(self, nbytes: int):
        ptr = ctypes.c_void_p()
        self.handle = (ctypes.c_ubyte * 64)()
        check(lib.q40_tp_alloc(nbytes, ctypes.byref(ptr), self.handle), "q40_tp_alloc")
        self.ptr, self.nbytes = int(ptr.value), nbytes

    @property
    def __cuda_array_interface__(self):
        return {"shape": (self.nbytes,), "typestr": "|u1", "data": (self.ptr, False), "version": 2}

    def as_tensor(self, device) -> torch.Tensor:
        return torch.as_tensor(self, device=device)

    def free(self):
        if self.ptr:
            lib.q40_tp_free(ctypes.c_void_p(self.ptr))
            self.ptr = 0


class PeerBuffers:
    """This rank's all-reduce buffer and the mapped buffers of the other ranks of `group`."""

    def __init__(self, rank: int, world: int, max_rows: int, dim: int, device, group=None):
        import torch.distributed as dist
        self.rank, self.world, self.max_rows, self.dim, self.device = rank, world, max_rows, dim, device
        self.group = group
        self.recv_off, total = layout(world, max_rows, dim)
        with torch.cuda.device(device):
            self.own = RawBuffer(total)
            handles = [None] * world
            dist.all_gather_object(handles, bytes(self.own.handle), group=group)
            self.ptrs = []
            for r in range(world):
                if r == rank:
                    self.ptrs.append(self.own.ptr)
                    continue
                p = ctypes.c_void_p()
                h = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
                check(lib.q40_tp_open(h, ctypes.byref(p)), "q40_tp_open")
                self.ptrs.append(int(p.value))
        self._arr = (ctypes.c_void_p * world)(*self.ptrs)
        dist.barrier(group=group)          # every buffer is zero-filled and mapped before the first push

    def allreduce_norm(self, partial: torch.Tensor, h: torch.Tensor, norm_w: Optional[torch.Tensor],
                       xn: Optional[torch.Tensor], eps: float, stream: int, wait_cycles: int = 0):
        rows, dim = h.shape
        check(lib.q40_tp_allreduce_norm(partial.data_ptr(), partial.stride(0), h.data_ptr(),
                                        norm_w.data_ptr() if norm_w is not None else None,
                                        xn.data_ptr() if xn is not None else None, rows, dim, float(eps), self.rank,
                                        self.world, self._arr, self.max_rows, int(wait_cycles), stream),
              "q40_tp_allreduce_norm")

    def status(self, clear: bool = False) -> int:
        """0 = every wait was met so far; 1 + r = rank r did not arrive in time in some call (synchronises)."""
        out = ctypes.c_int(0)
        st = torch.cuda.current_stream(self.device).cuda_stream
        check(lib.q40_tp_status(ctypes.c_void_p(self.own.ptr), ctypes.byref(out), 1 if clear else 0, st), "q40_tp_status")
        return int(out.value)

    def close(self):
        """Unmap the peers' buffers and free this rank's (collective: every rank calls it, none has a launch
        in flight that touches a peer)."""
        import torch.distributed as dist
        if not self.ptrs:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for r, p in enumerate(self.ptrs):
            if r != self.rank and p:
                lib.q40_tp_close(ctypes.c_void_p(p))
        dist.barrier(group=self.group)
        self.own.free()
        self.ptrs = []
