"""Peer-memory runtime: symmetric buffers shared between the ranks of one node.

Every rank allocates the same set of buffers with ``cudaMalloc`` (through the
native library), exports them as CUDA IPC handles, and maps its peers' buffers;
kernels then address ``ptrs[r]`` for any rank ``r``.  The handle exchange goes
through ``torch.distributed`` (any backend), so the same code runs under NCCL on
GPUs; the protocol logic is also exercised on CPU ranks with a stub allocator.

The reference shares memory between devices of ONE process through
``cuMemPoolSetAccess`` (backend/cuda/peer_linux.go:184-205); one process per GPU
needs IPC handles instead.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _native


class _RawCudaBuffer:
    """Exposes a raw device allocation to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2, "strides": None,
        }


class SymmetricBuffer:
    """One buffer per rank, same size everywhere; ``ptrs[r]`` is rank r's copy."""

    def __init__(self, nbytes: int, rank: int, world: int, group=None):
        lib = _native.lib()
        self.rank, self.world, self.nbytes = rank, world, nbytes
        out = ctypes.c_void_p()
        _native.check(lib.mimir_peer_alloc(nbytes, ctypes.byref(out)), "peer_alloc")
        self.local_ptr = out.value
        self._raw = _RawCudaBuffer(self.local_ptr, nbytes)
        self.bytes = torch.as_tensor(self._raw, device=f"cuda:{torch.cuda.current_device()}")
        self.ptrs = [0] * world
        self.ptrs[rank] = self.local_ptr
        self._opened = []
        if world > 1:
            handle = ctypes.create_string_buffer(64)
            _native.check(lib.mimir_ipc_export(ctypes.c_void_p(self.local_ptr), handle), "ipc_export")
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            for r in range(world):
                if r == rank:
                    continue
                p = ctypes.c_void_p()
                _native.check(lib.mimir_ipc_open(handles[r], ctypes.byref(p)), "ipc_open")
                self.ptrs[r] = p.value
                self._opened.append(p.value)

    def view(self, dtype: torch.dtype, offset_bytes: int = 0, numel: int | None = None) -> torch.Tensor:
        t = self.bytes[offset_bytes:]
        if numel is not None:
            t = t[: numel * torch.empty((), dtype=dtype).element_size()]
        return t.view(dtype)

    def ptr_array(self, offset_bytes: int = 0):
        arr = (ctypes.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.ptrs[r] + offset_bytes
        return arr

    def close(self) -> None:
        lib = _native.lib()
        for p in self._opened:
            lib.mimir_ipc_close(ctypes.c_void_p(p))
        self._opened = []
        if self.local_ptr:
            self.bytes = None
            self._raw = None
            lib.mimir_peer_free(ctypes.c_void_p(self.local_ptr))
            self.local_ptr = 0
