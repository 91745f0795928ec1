"""Symmetric heap: device buffers that every rank of a node maps into its own address space.

One process per GPU.  Each rank ``cudaMalloc``s its part, exports a CUDA IPC handle, the handles are
exchanged through ``torch.distributed`` (any backend; object all-gather) and every peer mapping is
opened once at set-up.  Kernels then receive a table of peer pointers and issue plain P2P loads /
stores (and ``multimem`` instructions when a multicast mapping is available) over NVLink.

The reference keeps per-GPU ``Signal`` buffers of ``sizeof(Signal) + max_elems·4`` bytes mapped with
peer access from ONE process (noeira/nn/distributed/process_group.mojo:182-216); here the same role
is played by IPC mappings across processes.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from .._native import check, cuda_lib

SIGNAL_PAD_WORDS = 64


class _RawCuda:
    """Minimal ``__cuda_array_interface__`` carrier so torch can view memory it did not allocate."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2,
                                         "strides": None}


class SymmetricBuffer:
    """``nbytes`` on every rank; ``local`` is a uint8 torch view, ``peer_ptrs[r]`` the address of rank
    r's part in THIS process (own address at ``[rank]``)."""

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None, solo: bool = False):
        """``solo`` keeps the buffer private to this process (world 1) even when a process group exists."""
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() and not solo else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() and not solo else 0
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        lib = cuda_lib()
        p = ctypes.c_void_p()
        check(lib.nb_symm_alloc(ctypes.byref(p), ctypes.c_longlong(self.nbytes)), "symm_alloc")
        self._own = p.value
        self.peer_ptrs: List[int] = [0] * self.world
        self.peer_ptrs[self.rank] = self._own
        self._opened = []
        if self.world > 1:
            h = (ctypes.c_ubyte * 64)()
            check(lib.nb_ipc_get_handle(ctypes.c_void_p(self._own), h), "ipc_get_handle")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(h), group=group)
            for r, hb in enumerate(handles):
                if r == self.rank:
                    continue
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(hb)
                q = ctypes.c_void_p()
                check(lib.nb_ipc_open_handle(buf, ctypes.byref(q)), f"ipc_open_handle(rank {r})")
                self.peer_ptrs[r] = q.value
                self._opened.append(q.value)
        self.local = torch.as_tensor(_RawCuda(self._own, self.nbytes), device=self.device)
        self.multicast_ptr = 0  # filled by `try_multicast`

    def view(self, dtype, offset_bytes: int = 0, numel: int = None) -> torch.Tensor:
        item = torch.empty((), dtype=dtype).element_size()
        n = (self.nbytes - offset_bytes) // item if numel is None else numel
        return self.local[offset_bytes: offset_bytes + n * item].view(dtype)

    def ptr_table(self, offset_bytes: int = 0):
        """ctypes array of ``world`` void* (peer addresses + offset) for a kernel launch."""
        arr = (ctypes.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.peer_ptrs[r] + offset_bytes
        return arr

    def close(self):
        lib = cuda_lib()
        for q in self._opened:
            lib.nb_ipc_close_handle(ctypes.c_void_p(q))
        self._opened = []
        if self._own:
            self.local = None
            lib.nb_symm_free(ctypes.c_void_p(self._own))
            self._own = 0


class SymmetricHeap:
    """Bump allocator over one SymmetricBuffer: sub-buffers share a single IPC mapping per peer."""

    def __init__(self, nbytes: int, group=None, solo: bool = False):
        self.buf = SymmetricBuffer(nbytes, group, solo=solo)
        self.off = 0
        self.world, self.rank = self.buf.world, self.buf.rank

    def alloc(self, nbytes: int, align: int = 256):
        o = (self.off + align - 1) // align * align
        if o + nbytes > self.buf.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {nbytes} at {o}, capacity {self.buf.nbytes}")
        self.off = o + nbytes
        return o

    def tensor(self, numel: int, dtype) -> "SymmTensor":
        item = torch.empty((), dtype=dtype).element_size()
        o = self.alloc(numel * item)
        return SymmTensor(self, o, numel, dtype)


class SymmTensor:
    def __init__(self, heap: SymmetricHeap, offset: int, numel: int, dtype):
        self.heap, self.offset, self.numel, self.dtype = heap, offset, numel, dtype
        self.local = heap.buf.view(dtype, offset, numel)

    def ptr_table(self):
        return self.heap.buf.ptr_table(self.offset)
