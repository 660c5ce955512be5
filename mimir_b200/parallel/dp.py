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
        # the full-size optimizer state of the single-GPU path is not needed any more; checkpoints go
        # through ``state_dict`` / ``load_state_dict`` below, which the engine delegates to
        engine.master = engine.exp_avg = engine.exp_avg_sq = None
        engine._dp = self
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

    # ----------------------------------------------------------- checkpoints
    def _gather_full(self, shard: torch.Tensor) -> torch.Tensor:
        """The full flat fp32 buffer assembled from every rank's slices, bucket by bucket."""
        e = self.engine
        full = torch.zeros(e.layout.total, dtype=torch.float32, device=e.device)
        for b in self.buckets.values():
            sl = b["count"] // self.world
            mine = shard[b["shard_off"]: b["shard_off"] + sl].contiguous()
            dst = full[b["start"]: b["start"] + b["count"]]
            if self.world > 1:
                dist.all_gather_into_tensor(dst, mine, group=self.group)
            else:
                dst.copy_(mine)
        return full

    def state_dict(self) -> dict:
        """Full tensors under the reference's checkpoint names (``model.<name>``, ``optim.<i>.exp_avg``,
        ``optim.<i>.exp_avg_sq``; train/checkpoint.go:40-73), the same on every rank: the optimizer
        state each rank owns is gathered bucket by bucket.  Collective: every rank must call it."""
        e = self.engine
        torch.cuda.current_stream().wait_stream(self.comm_stream)
        views = [e.layout.views(self._gather_full(t)) for t in (self.master, self.exp_avg, self.exp_avg_sq)]
        out = {}
        for i, name in enumerate(views[0]):
            out[f"model.{name}"] = views[0][name]
            out[f"optim.{i}.exp_avg"] = views[1][name]
            out[f"optim.{i}.exp_avg_sq"] = views[2][name]
        return out

    def load_state_dict(self, sd: dict) -> None:
        """Scatters a checkpoint written by ``state_dict`` (or by the single-device engine) back:
        every rank keeps its slices of the masters and moments and the whole bf16 parameter copy."""
        e = self.engine
        torch.cuda.current_stream().wait_stream(self.comm_stream)
        fulls = [torch.zeros(e.layout.total, dtype=torch.float32, device=e.device) for _ in range(3)]
        views = [e.layout.views(f) for f in fulls]
        for i, name in enumerate(views[0]):
            views[0][name].copy_(sd[f"model.{name}"])
            views[1][name].copy_(sd[f"optim.{i}.exp_avg"])
            views[2][name].copy_(sd[f"optim.{i}.exp_avg_sq"])
        for b in self.buckets.values():
            sl = b["count"] // self.world
            lo = b["start"] + sl * self.rank
            for full, shard in zip(fulls, (self.master, self.exp_avg, self.exp_avg_sq)):
                shard[b["shard_off"]: b["shard_off"] + sl].copy_(full[lo: lo + sl])
        e.params.copy_(fulls[0])
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)      # nobody reads a peer's parameters before all have loaded

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


class FusedFlatDataParallel:
    """Data parallelism for any ``nn`` model whose optimizer is on the fused flat AdamW path
    (``optim.FlatAdamW``): parameters and gradients live in peer-visible flat buffers, and after
    backward ONE kernel reduce-scatters the gradients by peer loads, applies AdamW to the slice this
    rank owns and all-gathers the new bf16 parameters by peer stores.  It replaces
    ``ReduceGrads`` + ``Step`` + ``BroadcastParams`` of the reference's ``train.Parallel``
    (train/parallel.go:226-286, 366-393); replicas stay bit-identical because every rank receives the
    same bytes.  Each rank keeps full-size moment buffers but updates only its slice;
    ``sync_state`` gathers the slices (in place) so that ``Optimizer.snapshot`` sees whole tensors."""

    def __init__(self, opt, group):
        from ..optim import FlatAdamW
        self.opt, self.group = opt, group
        self.rank, self.world = group.ranks.index(group.rank), group.size
        self.dp = FusedDataParallel(self.rank, self.world, torch.cuda.current_device(), group=group.pg)
        dev = opt.params[0]._data.device
        opt._flat = self.flat = FlatAdamW(opt, alloc=self.dp.alloc_shared, multiple=8 * self.world)
        n = self.flat.n
        self.sig = SymmetricBuffer(_SIG_WORDS * 4, self.rank, self.world, group.pg)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done_slots = torch.tensor([1], dtype=torch.int32, device=dev)
        self.shard = n // self.world
        pb, gb = self.dp._shared[0], self.dp._shared[1]
        self._params_arr, self._grads_arr, self._sig_arr = pb.ptr_array(), gb.ptr_array(), self.sig.ptr_array()
        # every replica starts from rank 0's weights
        dist.broadcast(self.flat.param, group.ranks[0], group=group.pg)
        dist.broadcast(self.flat.master, group.ranks[0], group=group.pg)
        self.nblocks = 2 * torch.cuda.get_device_properties(dev).multi_processor_count
        torch.cuda.synchronize()
        dist.barrier(group=group.pg)

    def begin(self) -> None:
        """Start of a step, before the forward pass reads the parameters: waits (on the device,
        bounded) until every peer has stored its slice of the previous update into this rank's
        parameter buffer, then opens the next epoch of the flag protocol."""
        _native.check(_native.lib().mimir_dp_step_begin(ptr(self.epoch), ctypes.c_void_p(self.sig.local_ptr), 1,
                                                        ptr(self.done_slots), self.world,
                                                        torch.cuda.current_stream().cuda_stream), "dp_step_begin")

    def step(self) -> None:
        """Reduce + AdamW + broadcast of one optimizer step (after ``begin`` and backward); the
        gradients are consumed."""
        opt, flat = self.opt, self.flat
        opt.steps += 1
        flat.stage(opt)
        flat.gather_grads()
        lib = _native.lib()
        st = torch.cuda.current_stream().cuda_stream
        h = opt.hyper
        rc = lib.mimir_dp_bucket(self._grads_arr, self._params_arr, self._sig_arr, ptr(flat.master), ptr(flat.exp_avg),
                                 ptr(flat.exp_avg_sq), ptr(flat.hyper), ptr(self.epoch), ptr(self.counter), 0, flat.n,
                                 flat.n, self.rank * self.shard, h.get("beta1", 0.9), h.get("beta2", 0.999),
                                 h.get("eps", 1e-8), opt.weight_decay, self.rank, self.world, 0, 1, self.nblocks, st)
        _native.check(rc, "dp_bucket")
        flat.bump()
        for p in flat.params:
            p._grad = None

    def sync_state(self) -> None:
        """Gathers every rank's slice of the masters and moments into the full buffers (in place)."""
        lo = self.rank * self.shard
        for buf in (self.flat.master, self.flat.exp_avg, self.flat.exp_avg_sq):
            dist.all_gather_into_tensor(buf, buf[lo: lo + self.shard], group=self.group.pg)

    def close(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(group=self.group.pg)
        # the parameters move back to ordinary memory before the shared buffers go away
        for p in self.flat.params:
            p._data = p._data.clone()
            p._grad, p._grad_buf = None, None
        self.opt._flat = None
        self.sync_state()
        index = {id(p): i for i, p in enumerate(self.opt.params)}
        for p in self.flat.params:
            st = self.opt.state[index[id(p)]]
            for k in ("master", "exp_avg", "exp_avg_sq"):
                st[k] = st[k].clone()
        self.sig.close()
        self.dp.close()


def fused_flat_eligible(opt, group) -> bool:
    """True when ``fit(data_parallel=group)`` can take the fused peer-memory path: NCCL ranks of one
    node, bf16 CUDA parameters, AdamW with master weights and no global-norm clip (the clip needs the
    norm of the reduced gradient before the update, which the one-pass kernel does not have)."""
    if not dist.is_initialized() or dist.get_backend(group.pg) != "nccl" or group.size < 2:
        return False
    return opt._flat is None and opt._flat_eligible() and not opt.clip_norm and opt.grad_scale == 1.0 \
        and group.size <= 8
