"""The public lazy tensor / nn / optim / train path on the native sm_100a kernels: a tiny GPT-2 built
from ``nn.DecoderBlock`` trains in bf16 through ``train.fit`` and matches fp32 PyTorch in losses and in
EVERY parameter's gradient, with no PyTorch library product / attention / normalisation / loss call."""
import contextlib

import pytest
import torch

pytestmark = pytest.mark.gpu

F = torch.nn.functional


@contextlib.contextmanager
def _no_library_ops():
    """Every PyTorch entry point the native kernels replace raises while this is active."""
    def trap(name, real):
        def f(*a, **k):
            if any(torch.is_tensor(x) and x.device.type == "meta" for x in a):
                return real(*a, **k)          # shape inference on meta tensors launches nothing
            raise AssertionError(f"library op {name} was called on the native path")
        return f
    saved = []
    for owner, name in [(F, "linear"), (F, "scaled_dot_product_attention"), (F, "layer_norm"), (F, "cross_entropy"),
                        (F, "gelu"), (F, "embedding"), (torch, "matmul"), (torch, "mm"), (torch, "bmm"),
                        (torch, "addmm"), (torch, "einsum"), (torch.Tensor, "__matmul__"), (torch.Tensor, "matmul")]:
        saved.append((owner, name, getattr(owner, name)))
        setattr(owner, name, trap(name, getattr(owner, name)))
    try:
        yield
    finally:
        for owner, name, fn in saved:
            setattr(owner, name, fn)


def _model(dtype=torch.bfloat16):
    import mimir_b200.tensor as T
    from mimir_b200 import nn
    from _tiny_gpt import TinyGPT
    nn.manual_seed(11)
    m = TinyGPT()
    ref = {n: p._data.clone().float() for n, p in m.named_params()}
    m.cast(dtype).to(T.GPU(0))
    return m, ref


def test_every_parameter_gets_its_gradient_from_the_native_kernels():
    import mimir_b200.tensor as T
    from mimir_b200 import _native
    from mimir_b200.ops._util import check_error_word
    from _tiny_gpt import loss_fn, torch_reference
    m, ref = _model()
    g = torch.Generator().manual_seed(5)
    tok = torch.randint(0, m.vocab, (4, 128), generator=g)
    tgt = torch.roll(tok, -1, 1)
    lib = _native.lib()
    n0 = lib.mimir_launch_count()
    with _no_library_ops():
        loss = loss_fn(m.vocab)(m(T.tensor(tok, device=T.GPU(0))), T.tensor(tgt, device=T.GPU(0)))
        loss.backward()
    assert lib.mimir_launch_count() - n0 >= 40          # the native kernels did the work
    assert check_error_word() == 0
    rp = {n: v.cuda().requires_grad_(True) for n, v in ref.items()}
    # the reference starts from the bf16-rounded weights the model really has
    with torch.no_grad():
        for n, p in m.named_params():
            rp[n].copy_(p._data.float())
    rl = torch_reference(m, rp, tok.cuda(), tgt.cuda())
    rl.backward()
    assert abs(loss.item() - rl.item()) < 3e-2, (loss.item(), rl.item())
    for n, p in m.named_params():
        assert p._grad is not None, f"{n} got no gradient"
        a, b = p._grad.float(), rp[n].grad
        err = (a - b).norm() / (b.norm() + 1e-12)
        assert err < 6e-2, (n, float(err))


def test_fit_trains_in_bf16_like_fp32_pytorch():
    import mimir_b200.tensor as T
    from mimir_b200 import data, optim
    from mimir_b200.ops._util import check_error_word
    from mimir_b200.tensor import plan
    from mimir_b200.train import fit
    from _tiny_gpt import loss_fn, torch_reference
    m, ref = _model()
    g = torch.Generator().manual_seed(6)
    tok = torch.randint(0, m.vocab, (40, 128), generator=g)
    tgt = torch.roll(tok, -1, 1)
    ds = data.Tensors(tok, tgt, batch_size=4, shuffle=False)
    opt = optim.AdamW(m.parameters(), lr=1e-3, weight_decay=0.01, master_weights=True, clip_norm=1.0)
    losses = []
    plan.clear_cache()
    before, unkeyed = plan.compiled(), plan.stats()["uncacheable"]
    with _no_library_ops():
        fit(m, opt, ds, loss=loss_fn(m.vocab), epochs=1, on_batch=lambda b: losses.append(b.loss), device=T.GPU(0))
    assert check_error_word() == 0
    assert opt._flat is not None, "AdamW with master weights did not take the fused flat path"
    assert plan.compiled() - before <= 4, plan.stats()          # ten steps: the step's schedule is planned once
                                                                # (plus the two host-to-device moves of a batch)
    assert plan.stats()["uncacheable"] == unkeyed               # every schedule of the loop had a structural key
    # fp32 PyTorch on the same data
    rp = {n: torch.nn.Parameter(v.to(torch.bfloat16).float().cuda()) for n, v in ref.items()}
    ropt = torch.optim.AdamW(rp.values(), lr=1e-3, weight_decay=0.01)
    rlosses = []
    for i in range(0, 40, 4):
        ropt.zero_grad()
        l = torch_reference(m, rp, tok[i:i + 4].cuda(), tgt[i:i + 4].cuda())
        l.backward()
        torch.nn.utils.clip_grad_norm_(rp.values(), 1.0)
        ropt.step()
        rlosses.append(l.item())
    assert len(losses) == 10
    for a, b in zip(losses, rlosses):
        assert abs(a - b) < 5e-2, (losses, rlosses)
    for n, p in m.named_params():
        d = (p._data.float() - rp[n].data).abs().max().item()
        assert d < 2e-2, (n, d)


def test_fit_replays_captured_steps_and_matches_the_eager_path():
    """Steps 4.. of ``fit`` run as CUDA-graph replays; the trained weights equal those of the same run
    with replay switched off (same kernels in the same order; the only difference two runs of the
    same program can show is the order of the embedding gradient's atomic adds, a bf16 ulp here and
    there)."""
    import os
    import mimir_b200.tensor as T
    from mimir_b200 import _native, data, optim
    from mimir_b200.ops._util import check_error_word
    from mimir_b200.train import fit
    from mimir_b200.train import replay as R
    from _tiny_gpt import loss_fn
    g = torch.Generator().manual_seed(8)
    tok = torch.randint(0, 512, (48, 128), generator=g)
    tgt = torch.roll(tok, -1, 1)
    results = []
    for graphs in ("1", "0"):
        os.environ["MIMIR_CUDA_GRAPHS"] = graphs
        m, _ = _model()
        ds = data.Tensors(tok, tgt, batch_size=4, shuffle=False)
        opt = optim.AdamW(m.parameters(), lr=1e-3, master_weights=True, clip_norm=1.0)
        seen = []
        made = []
        orig = R.StepReplay.__init__

        def spy(self, *a, **k):
            orig(self, *a, **k)
            made.append(self)
        R.StepReplay.__init__ = spy
        try:
            fit(m, opt, ds, loss=loss_fn(m.vocab), epochs=1, schedule=lambda e: 1e-3, on_batch=lambda b: seen.append(b.loss),
                device=T.GPU(0))
        finally:
            R.StepReplay.__init__ = orig
            os.environ.pop("MIMIR_CUDA_GRAPHS", None)
        assert check_error_word() == 0
        results.append(([p._data.clone() for p in m.parameters()], seen, made[0], opt.steps))
    (wa, la, ra, sa), (wb, lb, rb, sb) = results
    assert ra.captures == 1 and ra.replays == 12 - 3, (ra.captures, ra.replays)
    assert rb.captures == 0 and rb.replays == 0
    assert sa == sb == 12
    for x, y in zip(la, lb):
        assert abs(x - y) < 2e-3, (la, lb)
    for a, b in zip(wa, wb):          # at most a couple of bf16 ulps apart
        a, b = a.float(), b.float()
        assert bool(((a - b).abs() <= 2.0 ** -6 * a.abs() + 1e-3).all())
    assert _native.lib().mimir_launch_count() > 0


def test_llama_block_trains_through_native_rmsnorm_swiglu_and_gqa():
    import mimir_b200.tensor as T
    from mimir_b200 import nn
    from mimir_b200.ops._util import check_error_word
    nn.manual_seed(3)
    blk = nn.DecoderBlock(128, 2, hidden=256, kv_heads=1, style="llama")
    for p in blk.parameters():
        if p._data.dim() == 2:
            p._data.mul_(0.3)
    x = torch.randn(2, 128, 128) * 0.5
    want = []
    # fp32 CPU run of the same lazy code is the oracle
    out = blk(T.tensor(x, device=T.CPU()))
    T.mean(out * out).backward()
    want = {n: p._grad.clone() for n, p in blk.named_params()}
    lref = float(T.mean(out * out).item())
    blk.zero_grad()
    blk.cast(torch.bfloat16).to(T.GPU(0))
    with _no_library_ops():
        out = blk(T.tensor(x.to(torch.bfloat16), device=T.GPU(0)))
        l = T.mean(out * out)
        l.backward()
    assert check_error_word() == 0
    assert abs(l.item() - lref) < 3e-2 * max(1.0, abs(lref))
    for n, p in blk.named_params():
        assert p._grad is not None, n
        a, b = p._grad.float().cpu(), want[n]
        assert (a - b).norm() / (b.norm() + 1e-12) < 8e-2, n


def test_fit_data_parallel_on_two_gpus_equals_one_gpu():
    """``fit(data_parallel=)`` takes the fused reduce + AdamW + broadcast kernel; two ranks on halves of
    every batch end where one device ends on the whole batch, replicas bit-identical, optimizer state
    whole again after the run."""
    import json
    import os
    import subprocess
    import sys
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29561", os.path.join(here, "_public_dp_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-3000:]
    res = [json.loads(l[7:]) for l in out.stdout.splitlines() if l.startswith("RESULT ")]
    assert len(res) == 2
    for r in res:
        assert r["err"] == 0 and r["identical"] and r["steps"] == 8, r
    r0 = [r for r in res if r["rank"] == 0][0]
    for a, b in zip(r0["loss"], r0["single_loss"]):
        assert abs(a - b) < 3e-2, r0
    assert r0["max_param_diff"] < 1e-2 and r0["moment_diff"] < 1e-2, r0
