"""Symmetric communication arena: one cudaMalloc per rank, mapped by every peer through CUDA IPC.

Every rank lays its arena out identically (flags | scalars | counters | named regions), so a
region has the same byte offset on all ranks and a kernel addresses rank r's copy as
``peer_base[r] + offset``.  ``torch.distributed`` is used only to exchange the 64-byte IPC
handles at start-up.  Tensors over arena memory are created zero-copy through the CUDA array
interface.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib

_HDR_FLAGS = 1024       # flag words (NUM_FLAG_KINDS x MAX_RANKS uint32), padded
_HDR_SCALARS = 1024     # 2 x MAX_RANKS floats, padded
_HDR_COUNTERS = 1024    # 256 uint32 launch counters (local use)
_HEADER = _HDR_FLAGS + _HDR_SCALARS + _HDR_COUNTERS


class _CudaMem:
    """Minimal CUDA-array-interface carrier so torch can wrap raw device memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def _wrap(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.as_tensor(_CudaMem(ptr, nbytes), device=device)


class SymmetricArena:
    def __init__(self, regions: List[Tuple[str, int]], rank: int, world_size: int, device: torch.device,
                 group=None):
        """``regions``: (name, nbytes) in layout order; identical on every rank."""
        self.rank, self.world_size, self.device = rank, world_size, device
        L = _lib.lib()
        L.llmb_comm_alloc.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_longlong]
        L.llmb_ipc_get_handle.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        L.llmb_ipc_open.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
        L.llmb_ipc_close.argtypes = [ctypes.c_void_p]
        L.llmb_comm_free.argtypes = [ctypes.c_void_p]
        self.offsets: Dict[str, int] = {}
        self.sizes: Dict[str, int] = {}
        off = _HEADER
        for name, nbytes in regions:
            off = (off + 1023) // 1024 * 1024
            self.offsets[name], self.sizes[name] = off, nbytes
            off += nbytes
        self.nbytes = (off + 1023) // 1024 * 1024
        base = ctypes.c_void_p()
        _lib.check(L.llmb_comm_alloc(ctypes.byref(base), self.nbytes), "comm_alloc")
        self.base = base.value
        self.peer_bases: List[int] = [0] * world_size
        self.peer_bases[rank] = self.base
        self._opened: List[int] = []
        if world_size > 1:
            handle = ctypes.create_string_buffer(64)
            _lib.check(L.llmb_ipc_get_handle(self.base, handle), "ipc_get_handle")
            gathered: List[Optional[bytes]] = [None] * world_size
            dist.all_gather_object(gathered, (bytes(handle.raw), torch.cuda.current_device()), group=group)
            for r, (h, dev) in enumerate(gathered):
                if r == rank:
                    continue
                p = ctypes.c_void_p()
                buf = ctypes.create_string_buffer(h, 64)
                _lib.check(L.llmb_ipc_open(ctypes.byref(p), buf), f"ipc_open(rank {r})")
                self.peer_bases[r] = p.value
                self._opened.append(p.value)
            dist.barrier(group=group)
        self._mem = _wrap(self.base, self.nbytes, device)

    # -- views ---------------------------------------------------------------------------------
    def tensor(self, name: str, dtype: torch.dtype) -> torch.Tensor:
        off, n = self.offsets[name], self.sizes[name]
        return self._mem[off:off + n].view(dtype)

    def peer_ptrs(self, name: Optional[str] = None, extra: int = 0):
        """ctypes array of W pointers to region ``name`` (or the arena base) on every rank."""
        off = (self.offsets[name] if name else 0) + extra
        arr = (ctypes.c_void_p * 8)()
        for r in range(self.world_size):
            arr[r] = self.peer_bases[r] + off
        return arr

    @property
    def flags_ptr(self) -> int:
        return self.base

    @property
    def scalars_ptr(self) -> int:
        return self.base + _HDR_FLAGS

    def counter_ptr(self, i: int) -> int:
        return self.base + _HDR_FLAGS + _HDR_SCALARS + 4 * i

    def flags_peer_ptrs(self):
        return self.peer_ptrs(None, 0)

    def scalars_peer_ptrs(self):
        return self.peer_ptrs(None, _HDR_FLAGS)

    def close(self) -> None:
        L = _lib.lib()
        self._mem = None
        for p in self._opened:
            L.llmb_ipc_close(p)
        self._opened = []
        if self.base:
            L.llmb_comm_free(self.base)
            self.base = 0
