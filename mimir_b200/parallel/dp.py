"""Data-parallel training with the gradient reduce, the AdamW update and the
parameter broadcast fused into one peer-memory kernel per bucket, overlapped
with backward (``csrc/comm.cu``).

Covers the reference's ``train.Parallel`` (train/parallel.go:78-286,366-393) and
``Group.ReduceGrads / AllReduceGrads / BroadcastParams`` (tensor/group.go:285-478)
for the kernel-sequence engines: same result as single-device training on the
concatenated batch (each share's loss is the mean over its rows and gradients
are averaged over ranks, train/parallel.go:231-234), bit-identical replicas.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _native
from ..ops._util import ptr
from .peer import SymmetricBuffer

_SIG_WORDS = 4096


class FusedDataParallel:
    def __init__(self, rank: int, world: int, local_rank: int | None = None, nblocks: int = 0,
                 group=None):
        self.rank, self.world, self.group = rank, world, group
        self.local_rank = rank if local_rank is None else local_rank
        self.nblocks = nblocks
        self._shared = []  # SymmetricBuffer for params, grads (in allocation order)
        self.engine = None
        self.comm_stream = None

    # The engine calls this for its flat parameter and gradient buffers.
    def alloc_shared(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        buf = SymmetricBuffer(nbytes, self.rank, self.world, self.group)
        self._shared.append(buf)
        return buf.view(dtype, 0, numel)

    def attach(self, engine) -> None:
        """Shards the optimizer state and prepares per-bucket launch arguments."""
        if len(self._shared) < 2:
            raise RuntimeError("engine must allocate params and grads through alloc_shared")
        self.engine = engine
        w = self.world
        self.param_buf, self.grad_buf = self._shared[0], self._shared[1]
        self.sig_buf = SymmetricBuffer(_SIG_WORDS * 4, self.rank, w, self.group)
        dev = engine.device
        total = engine.layout.total
        if total % (8 * w):
            raise ValueError("flat parameter buffer must be divisible by 8 * world")
        # every replica must start from the same weights: rank 0's
        if w > 1:
            dist.broadcast(engine.params, 0, group=self.group)
            dist.broadcast(engine.master, 0, group=self.group)
        shard = total // w
        self.master = torch.empty(shard, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(shard, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(shard, dtype=torch.float32, device=dev)
        self.buckets = {}
        off = 0
        for i, (name, start, decay_n, count) in enumerate(engine.layout.buckets):
            sl = count // w
            self.master[off:off + sl].copy_(engine.master[start + sl * self.rank: start + sl * (self.rank + 1)])
            self.buckets[name] = dict(start=start, count=count, decay_n=decay_n, shard_off=off,
                                      slot_ready=2 * i, slot_done=2 * i + 1)
            off += sl
        # the full-size optimizer state of the single-GPU path is not needed any more
        engine.master = engine.exp_avg = engine.exp_avg_sq = None
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.block_counters = torch.zeros(len(self.buckets), dtype=torch.int32, device=dev)
        self.done_slots = torch.tensor([b["slot_done"] for b in self.buckets.values()],
                                       dtype=torch.int32, device=dev)
        self.comm_stream = torch.cuda.Stream(device=dev)
        self._grads_arr = self.grad_buf.ptr_array()
        self._params_arr = self.param_buf.ptr_array()
        self._sig_arr = self.sig_buf.ptr_array()
        self._bucket_index = {n: i for i, n in enumerate(self.buckets)}
        self._last_bucket = engine.layout.buckets[0][0]   # backward finishes the buckets in reverse layout order
        if w > 1:
            dist.barrier(group=self.group)
        torch.cuda.synchronize()

    # ----------------------------------------------------------------- step
    def begin_step(self) -> None:
        lib = _native.lib()
        _native.check(lib.mimir_dp_step_begin(ptr(self.epoch), ctypes.c_void_p(self.sig_buf.local_ptr),
                                              len(self.buckets), ptr(self.done_slots), self.world,
                                              torch.cuda.current_stream().cuda_stream), "dp_step_begin")

    def on_bucket_ready(self, name: str, betas, eps, wd) -> None:
        """Called by backward when the gradients of bucket ``name`` are final."""
        main = torch.cuda.current_stream()
        self.comm_stream.wait_stream(main)
        b = self.buckets[name]
        e = self.engine
        lib = _native.lib()
        # Two small blocks per SM (nblocks = 0): the bucket kernel is latency-bound per thread, so a
        # narrow grid falls behind backward and the backlog surfaces at the end of the step (GPT-2 small
        # on 2 GPUs: 15.5 / 13.2 / 12.7 / 12.3 / 12.1 ms per step with 8 / 16 / 32 / 64 / 296 blocks);
        # its blocks hold no shared memory and sit beside the GEMM CTAs.  The last bucket of the step
        # has the GPU to itself and always takes the full grid.
        last = name == self._last_bucket
        full = 2 * torch.cuda.get_device_properties(e.device).multi_processor_count
        nblocks = full if last or self.nblocks <= 0 else self.nblocks
        rc = lib.mimir_dp_bucket(self._grads_arr, self._params_arr, self._sig_arr, ptr(self.master),
                                 ptr(self.exp_avg), ptr(self.exp_avg_sq), ptr(e.hyper), ptr(self.epoch),
                                 self.block_counters[self._bucket_index[name]:].data_ptr(), b["start"],
                                 b["count"], b["decay_n"], b["shard_off"], betas[0], betas[1], eps, wd,
                                 self.rank, self.world, b["slot_ready"], b["slot_done"], nblocks,
                                 self.comm_stream.cuda_stream)
        _native.check(rc, "dp_bucket")

    def run_backward_and_update(self, trainer) -> None:
        e = self.engine
        e.backward(on_bucket_ready=lambda n: self.on_bucket_ready(n, trainer.betas, trainer.eps, trainer.wd))
        torch.cuda.current_stream().wait_stream(self.comm_stream)

    def close(self) -> None:
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        for b in (getattr(self, "sig_buf", None), *self._shared):
            if b is not None:
                b.close()
        self._shared = []
