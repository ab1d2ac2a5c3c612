"""Symmetric heap: one device allocation per rank, mapped into every peer of the group.

Each rank cudaMallocs a heap of the same size, exports a CUDA IPC handle, and opens the handles of
the others (exchanged through torch.distributed). After that `ptrs[r]` is an address that THIS
process can hand to a kernel to read or write rank r's heap over NVLink; `ptrs[rank]` is the local
heap. Regions are carved out with `alloc`, at identical offsets on every rank, so a region's
address on peer r is `ptrs[r] + offset`.

With `multicast=True` the heap is instead allocated through torch's symmetric-memory allocator (CUDA VMM
handles exchanged between the processes), which also binds all ranks' heaps to one NVLink multicast object:
`mc_ptr + offset` then addresses the same region on every rank at once, for `multimem` loads that the NVSwitch
reduces (csrc/kernels/norm.cu). A rank must not die while its heap is bound to a multicast object (the switch
faults its peers), so the failure-handling tests and every run that may lose a rank use the plain heap.

The reference's counterpart is the file rendezvous of the NCCL id plus a host shared-memory segment
for its 2-rank all-reduce (crates/skein_runtime/src/distributed/rendezvous.rs:19,48;
crates/skein_runtime/src/cuda/shm_allreduce.rs:85); here the shared segment is device memory.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib


class _DevMem:
    """Exposes a raw device pointer through __cuda_array_interface__ so torch can view it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class SymmetricHeap:
    def __init__(self, group, device: torch.device, nbytes: int, multicast: bool = False):
        self.group = group
        self.device = device
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self.nbytes = (nbytes + 255) // 256 * 256
        self.mc_ptr = 0
        self._cursor = 0
        self._opened = []
        self._symm = None
        if multicast:
            import torch.distributed._symmetric_memory as symm_mem
            self._symm = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
            self._symm.zero_()
            self._hdl = symm_mem.rendezvous(self._symm, group)
            self.ptrs = [int(q) for q in self._hdl.buffer_ptrs]
            self.mc_ptr = int(self._hdl.multicast_ptr)
            if not self.mc_ptr:
                raise RuntimeError("this group has no NVLink multicast support (multicast_ptr is null)")
            self.local_ptr = self.ptrs[self.rank]
            if self.local_ptr != self._symm.data_ptr():
                raise RuntimeError("symmetric-memory rendezvous returned a different address for the local heap")
            self.local = self._symm
            torch.cuda.synchronize(device)
            dist.barrier(group=group)
            return
        L = _lib.lib()
        p = C.c_void_p()
        _lib.check(L.skein_ipc_alloc(C.byref(p), self.nbytes), "ipc_alloc")
        self.local_ptr = p.value
        hb = L.skein_ipc_handle_bytes()
        buf = C.create_string_buffer(hb)
        _lib.check(L.skein_ipc_get_handle(self.local_ptr, buf), "ipc_get_handle")
        handles = [None] * self.size
        dist.all_gather_object(handles, bytes(buf.raw), group=group)
        self.ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local_ptr)
                continue
            q = C.c_void_p()
            _lib.check(L.skein_ipc_open(C.create_string_buffer(h, hb), C.byref(q)), f"ipc_open(rank {r})")
            self.ptrs.append(q.value)
            self._opened.append(q.value)
        self._holder = _DevMem(self.local_ptr, self.nbytes)
        self.local = torch.as_tensor(self._holder, device=device)  # uint8 view of the local heap
        dist.barrier(group=group)

    def alloc(self, nbytes: int, align: int = 256) -> int:
        """Reserve a region; returns its offset (identical on every rank if all ranks call in the same order)."""
        off = (self._cursor + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted ({off + nbytes} > {self.nbytes})")
        self._cursor = off + nbytes
        return off

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        return self.local[offset:offset + nb].view(dtype).view(*shape)

    def peer_ptr(self, r: int, offset: int) -> int:
        return self.ptrs[r] + offset

    def mc_addr(self, offset: int) -> int:
        """Multicast address of a region (0 when the heap has no multicast mapping)."""
        return self.mc_ptr + offset if self.mc_ptr else 0

    def close(self):
        if self._symm is not None:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)      # nobody unbinds while a peer may still read through the switch
            self.local, self._hdl, self._symm, self.local_ptr = None, None, None, None
            return
        L = _lib.lib()
        for q in self._opened:
            L.skein_ipc_close(q)
        self._opened = []
        if self.local_ptr:
            self.local = None
            L.skein_ipc_free(self.local_ptr)
            self.local_ptr = None
