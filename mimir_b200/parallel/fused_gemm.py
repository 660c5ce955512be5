"""GEMMs fused with their collective (``csrc/gemm_comm_sm100.cu``).

``AllGatherLinear``: y = x W^T with W sharded by output rows over the ranks (a
fully sharded or column-parallel weight); the all-gather runs inside the GEMM
kernel.  ``ReduceScatterGemm``: out = reduce_scatter(A B^T) along the rows of the
product (row-parallel layers, sharded weight gradients); finished tiles leave for
their owner while the rest of the product is still being computed.
The NCCL lowering of the same two patterns (``all_gather`` + GEMM, GEMM +
``reduce_scatter``) is kept as ``*_baseline`` for tests and comparisons
(reference: tensor/reshard.go:242-336).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _native
from ..ops._util import ptr, stream_ptr
from ..ops.gemm import GEMM_FLAGS, gemm
from .peer import SymmetricBuffer

_declared = False


def _L():
    global _declared
    lib = _native.lib()
    if not _declared:
        P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        PP = ctypes.POINTER(ctypes.c_void_p)
        lib.mimir_gemm_allgather_b.restype = I
        lib.mimir_gemm_allgather_b.argtypes = [P, PP, P, I, I, I, I, I, P, P, I, P, I, P, P, P, I, I, P]
        lib.mimir_gemm_reduce_scatter.restype = I
        lib.mimir_gemm_reduce_scatter.argtypes = [P, P, I, I, I, I, I, I, I, PP, PP, P, P, P, I, I, I, P]
        lib.mimir_comm_set_peer_wait_ms.argtypes = [L]
        lib.mimir_comm_set_peer_wait_ms.restype = None
        _declared = True
    return lib


class ShardedWeight:
    """A weight [N, K] sharded by rows: every rank holds a full-size symmetric buffer and
    keeps its own rows current in it; the other rows are scratch the fused GEMM fills."""

    def __init__(self, N: int, K: int, rank: int, world: int, group=None, arena: SymmetricBuffer | None = None,
                 offset: int = 0):
        """``arena`` / ``offset`` place the matrix inside an existing symmetric buffer (one allocation and
        one handle exchange for a whole model) instead of a buffer of its own."""
        if N % world:
            raise ValueError("rows must divide by the number of ranks")
        if offset % 16:
            raise ValueError("the matrix must start on a 16-byte boundary of the arena")
        self.N, self.K, self.rank, self.world = N, K, rank, world
        self._own_buf = arena is None
        self.buf = SymmetricBuffer(N * K * 2, rank, world, group) if arena is None else arena
        self.full = self.buf.view(torch.bfloat16, offset, N * K).view(N, K)
        self.rows = N // world
        self.shard = self.full[rank * self.rows: (rank + 1) * self.rows]
        dev = self.full.device
        self.state = torch.zeros(world + 2, dtype=torch.int32, device=dev)  # shard counters, epoch, done
        self._arr = self.buf.ptr_array(offset)

    def close(self):
        if self._own_buf:
            self.buf.close()


def gemm_allgather(x: torch.Tensor, w: ShardedWeight, out=None, bias=None, gelu=False, residual=False, aux=None):
    """``x [M,K] @ gather(w)^T`` with the gather inside the kernel.  Peers must not be
    writing their shards while this runs (separate optimizer steps with a barrier)."""
    M, K = x.shape
    if out is None:
        out = torch.empty(M, w.N, dtype=torch.bfloat16, device=x.device)
    flags = (GEMM_FLAGS["gelu"] if gelu else 0) | (GEMM_FLAGS["residual"] if residual else 0)
    st = w.state
    rc = _L().mimir_gemm_allgather_b(ptr(x), w._arr, ptr(out), M, w.N, K, x.stride(0), out.stride(0), ptr(bias),
                                     ptr(aux), aux.stride(0) if aux is not None else 0, None, flags,
                                     st.data_ptr(), st[w.world:].data_ptr(), st[w.world + 1:].data_ptr(), w.rank,
                                     w.world, stream_ptr())
    _native.check(rc, "gemm_allgather")
    return out


def gemm_allgather_baseline(x, w: ShardedWeight, group=None):
    parts = [torch.empty_like(w.shard) for _ in range(w.world)]
    dist.all_gather(parts, w.shard.contiguous(), group=group)
    return gemm(x, torch.cat(parts, 0))


class ReduceScatterGemm:
    """State of one reduce-scatter call site: staging slabs [world][M/world][N] and flags.

    Calls on one object may follow each other directly (same stream on every rank, no host barrier
    and no other collective in between): a rank publishes "I have summed call k" to its peers, and
    the kernel of call k+1 waits for the owner's flag before its first store into that owner's slabs.
    Two objects never share slabs, so calls on different objects are independent.  The ranks must
    issue the calls of one object in the same order."""

    def __init__(self, M: int, N: int, rank: int, world: int, group=None, slot: int = 0):
        if M % world or (M // world) % 32:
            raise ValueError("rows per rank must be a multiple of 32")
        self.M, self.N, self.rank, self.world, self.slot = M, N, rank, world, slot
        self.stage = SymmetricBuffer(M * N * 2, rank, world, group)
        self.sig = SymmetricBuffer(1024 * 4, rank, world, group)
        dev = self.stage.bytes.device
        self.state = torch.zeros(2, dtype=torch.int32, device=dev)
        self._stage_arr, self._sig_arr = self.stage.ptr_array(), self.sig.ptr_array()

    def __call__(self, a: torch.Tensor, b: torch.Tensor, transposed: bool = False, out=None, b_mn: bool | None = None):
        """``a [M,K] @ b[N,K]^T`` (or, ``transposed``, a stored [K,M] and b stored [K,N]; or, with
        ``b_mn`` alone, a [M,K] and b stored [K,N]): returns this rank's rows ``[M/world, N]`` of the
        sum over ranks."""
        if transposed:
            K, M = a.shape
        else:
            M, K = a.shape
        b_mn = transposed if b_mn is None else b_mn
        if out is None:
            out = torch.empty(M // self.world, self.N, dtype=torch.bfloat16, device=a.device)
        rc = _L().mimir_gemm_reduce_scatter(ptr(a), ptr(b), M, self.N, K, a.stride(0), b.stride(0), int(transposed),
                                            int(b_mn), self._stage_arr, self._sig_arr, ptr(out),
                                            self.state.data_ptr(), self.state[1:].data_ptr(), self.rank, self.world,
                                            self.slot, stream_ptr())
        _native.check(rc, "gemm_reduce_scatter")
        return out

    def close(self):
        self.stage.close()
        self.sig.close()


def gemm_reduce_scatter_baseline(a, b, world, transposed=False, group=None):
    full = gemm(a, b, a_mn=transposed, b_mn=transposed)
    out = torch.empty(full.shape[0] // world, full.shape[1], dtype=full.dtype, device=full.device)
    dist.reduce_scatter_tensor(out, full, group=group)
    return out
