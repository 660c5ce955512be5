"""Row / elementwise kernels against plain fp32 PyTorch on the same bf16 inputs."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
F = torch.nn.functional


def close(a, b, tol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    assert err <= tol * (b.abs().max().item() + 1e-3), f"err {err}"


@pytest.mark.parametrize("rows,C", [(37, 768), (64, 256), (9, 1024), (16, 2048), (5, 136)])
def test_layernorm_fwd_bwd(rows, C):
    from mimir_b200.ops import kernels as K
    torch.manual_seed(0)
    x = torch.randn(rows, C, device="cuda").bfloat16()
    g = (1 + 0.1 * torch.randn(C, device="cuda")).bfloat16()
    b = (0.1 * torch.randn(C, device="cuda")).bfloat16()
    dy = torch.randn(rows, C, device="cuda").bfloat16()
    dres = torch.randn(rows, C, device="cuda").bfloat16()
    y = torch.empty_like(x)
    mean = torch.empty(rows, device="cuda")
    rstd = torch.empty(rows, device="cuda")
    K.layernorm_fwd(x, g, b, y, mean, rstd)
    xr = x.float().requires_grad_(True)
    gr = g.float().requires_grad_(True)
    br = b.float().requires_grad_(True)
    yr = F.layer_norm(xr, (C,), gr, br, 1e-5)
    close(y, yr)
    yr.backward(dy.float())
    dx = torch.empty_like(x)
    dg = torch.empty_like(g)
    db = torch.empty_like(b)
    K.layernorm_bwd(dy, x, g, mean, rstd, dres, dx, dg, db, K.norm_bwd_scratch(C, x.device))
    close(dx, xr.grad + dres.float())
    close(dg, gr.grad, 3e-2)
    close(db, br.grad, 3e-2)


@pytest.mark.parametrize("rows,C", [(33, 2048), (7, 512)])
def test_rmsnorm_fwd_bwd(rows, C):
    from mimir_b200.ops import kernels as K
    torch.manual_seed(1)
    x = torch.randn(rows, C, device="cuda").bfloat16()
    g = (1 + 0.1 * torch.randn(C, device="cuda")).bfloat16()
    dy = torch.randn(rows, C, device="cuda").bfloat16()
    y = torch.empty_like(x)
    rstd = torch.empty(rows, device="cuda")
    K.rmsnorm_fwd(x, g, y, rstd, 1e-6)
    xr = x.float().requires_grad_(True)
    gr = g.float().requires_grad_(True)
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * gr
    close(y, yr)
    yr.backward(dy.float())
    dx = torch.empty_like(x)
    dg = torch.empty_like(g)
    K.rmsnorm_bwd(dy, x, g, rstd, None, dx, dg, K.norm_bwd_scratch(C, x.device))
    close(dx, xr.grad)
    close(dg, gr.grad, 3e-2)


@pytest.mark.parametrize("rows,V,Vp", [(50, 1000, 1024), (9, 16384, 16384), (7, 32000, 32000), (5, 50257, 50304),
                                       (3, 65536, 65536), (3, 70001, 70016), (2, 128256, 128256)])
def test_cross_entropy_padded_vocab(rows, V, Vp):
    """Vocabularies from 1000 to 128256 columns, padded or not, in place, out of place and loss only."""
    from mimir_b200.ops import kernels as K
    torch.manual_seed(2)
    logits = torch.randn(rows, Vp, device="cuda").bfloat16() * 3
    tgt = torch.randint(0, V, (rows,), device="cuda")
    tgt[min(3, rows - 1)] = -100
    lr = logits[:, :V].float().requires_grad_(True)
    ref = F.cross_entropy(lr, tgt, ignore_index=-100, reduction="sum") / rows
    ref.backward()
    loss_rows = torch.empty(rows, device="cuda")
    mean = torch.zeros(1, device="cuda")
    work = logits.clone()
    K.cross_entropy(work, tgt, loss_rows, work, mean, V, 1.0 / rows, 1.0 / rows)
    assert abs(mean.item() - ref.item()) < 2e-2 * abs(ref.item())
    close(work[:, :V], lr.grad, 3e-2)
    if Vp > V:
        assert work[:, V:].abs().max().item() == 0
    # not in place, and loss only
    out = torch.full_like(logits, 7.0)
    K.cross_entropy(logits, tgt, loss_rows, out, mean, V, 1.0 / rows, 1.0 / rows)
    assert torch.equal(out, work)
    loss2 = torch.empty(rows, device="cuda")
    K.cross_entropy(logits, tgt, loss2, None, None, V, 1.0, 1.0)
    assert torch.equal(loss2, loss_rows)


def test_colsum_embedding_adamw():
    from mimir_b200.ops import kernels as K
    torch.manual_seed(3)
    x = torch.randn(1000, 776, device="cuda").bfloat16()
    out = torch.empty(776, device="cuda", dtype=torch.bfloat16)
    K.colsum(x, out, torch.empty(64 * 776, device="cuda"))
    close(out, x.float().sum(0), 2e-2)
    # embedding
    V, C, B, T = 100, 64, 3, 16
    wte = torch.randn(V, C, device="cuda").bfloat16()
    wpe = torch.randn(T, C, device="cuda").bfloat16()
    tok = torch.randint(0, V, (B * T,), device="cuda")
    o = torch.empty(B * T, C, device="cuda", dtype=torch.bfloat16)
    K.embedding_fwd(tok, wte, wpe, o, T)
    close(o, wte.float()[tok] + wpe.float().repeat(B, 1))
    dx = torch.randn(B * T, C, device="cuda").bfloat16()
    dwte = torch.zeros_like(wte)
    dwpe = torch.zeros_like(wpe)
    K.embedding_bwd(tok, dx, dwte, dwpe, B, T)
    ref = torch.zeros(V, C, device="cuda").index_add_(0, tok, dx.float())
    close(dwte, ref, 3e-2)
    close(dwpe, dx.float().view(B, T, C).sum(0))
    # adamw against the rule of optim/optim.go:494-510
    n = 4096
    master = torch.randn(n, device="cuda")
    p0 = master.clone()
    grad = torch.randn(n, device="cuda").bfloat16()
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    param = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
    for step in (1, 2, 3):
        K.adamw_flat(master, param, grad, m, v, decay_n=2048, lr=lr, beta1=b1, beta2=b2, eps=eps,
                     wd=wd, step=step)
    p, mm, vv = p0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    g = grad.float()
    wdv = torch.cat([torch.full((2048,), wd), torch.zeros(n - 2048)]).cuda()
    for step in (1, 2, 3):
        p = p * (1 - lr * wdv)
        mm = b1 * mm + (1 - b1) * g
        vv = b2 * vv + (1 - b2) * g * g
        p = p - (lr / (1 - b1 ** step)) * mm / (vv.sqrt() / math.sqrt(1 - b2 ** step) + eps)
    assert (master - p).abs().max().item() < 1e-5
    close(param, p)


def test_swiglu_rope_act():
    from mimir_b200.ops import kernels as K
    torch.manual_seed(4)
    rows, Fd = 40, 128
    gu = torch.randn(rows, 2 * Fd, device="cuda").bfloat16()
    y = torch.empty(rows, Fd, device="cuda", dtype=torch.bfloat16)
    K.swiglu_fwd(gu, y)
    gr = gu.float().requires_grad_(True)
    ref = F.silu(gr[:, :Fd]) * gr[:, Fd:]
    close(y, ref)
    dy = torch.randn_like(y)
    ref.backward(dy.float())
    dgu = torch.empty_like(gu)
    K.swiglu_bwd(gu, dy, dgu)
    close(dgu, gr.grad)
    # rope halves order
    H, D = 2, 32
    x = torch.randn(rows, H * D, device="cuda").bfloat16()
    pos = torch.arange(rows, device="cuda", dtype=torch.int32)
    freqs = (1.0 / 10000 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    x0 = x.clone()
    K.rope_(x, pos, freqs, 0, H, D, interleaved=False)
    ang = pos.float()[:, None] * freqs[None]
    xf = x0.float().view(rows, H, D)
    a, b = xf[..., : D // 2], xf[..., D // 2:]
    ref = torch.cat([a * ang.cos()[:, None] - b * ang.sin()[:, None],
                     a * ang.sin()[:, None] + b * ang.cos()[:, None]], -1).view(rows, H * D)
    close(x, ref)
    K.rope_(x, pos, freqs, 0, H, D, interleaved=False, inverse=True)
    close(x, x0.float(), 3e-2)


def test_philox_kernel_matches_host_stream_bit_for_bit():
    from mimir_b200.ops import kernels as K
    from mimir_b200.tensor.random import philox_uniform
    for n, seed in ((1, 0), (1027, 42), (65536, 0x1234567890ABCDEF)):
        got = K.philox_uniform(n, seed).cpu()
        want = philox_uniform((n,), seed, "cpu")
        assert torch.equal(got, want)
    x = torch.randn(4099, device="cuda").bfloat16()
    y = K.dropout(x, 0.25, 7)
    keep = philox_uniform((4099,), 7, "cpu") >= 0.25
    ref = torch.where(keep.cuda(), (x.float() / 0.75).bfloat16(), torch.zeros_like(x))
    assert torch.equal(y, ref)
    assert torch.equal(K.dropout(x, 0.25, 7), y)


@pytest.mark.parametrize("mode", ["sum", "max", "logsumexp"])
@pytest.mark.parametrize("shape,dim,dtype", [((5, 37), -1, torch.float32), ((3, 1024), -1, torch.float32),
                                             ((2, 5000), 1, torch.float32), ((4, 300, 6), 1, torch.float32),
                                             ((7, 2050), -1, torch.bfloat16), ((1, 1), 0, torch.float32)])
def test_scan_rows_against_torch(mode, shape, dim, dtype):
    from mimir_b200.ops.scan import scan
    torch.manual_seed(sum(shape))
    x = torch.randn(*shape).to(dtype)
    ref = {"sum": lambda v: torch.cumsum(v, dim), "max": lambda v: torch.cummax(v, dim).values,
           "logsumexp": lambda v: torch.logcumsumexp(v, dim)}[mode](x.double())
    got = scan(x.cuda(), mode, dim)
    assert got.dtype == dtype and got.shape == x.shape
    tol = dict(rtol=2e-2, atol=0.5) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(got.double().cpu(), ref, **tol)
    rev = scan(x.cuda(), mode, dim, reverse=True)
    ref_r = {"sum": lambda v: torch.cumsum(v, dim), "max": lambda v: torch.cummax(v, dim).values,
             "logsumexp": lambda v: torch.logcumsumexp(v, dim)}[mode](x.double().flip(dim)).flip(dim)
    torch.testing.assert_close(rev.double().cpu(), ref_r, **tol)


def test_lazy_scans_use_the_native_kernel_on_the_gpu():
    from mimir_b200 import tensor as T
    x = torch.randn(6, 777)
    for f, ref in ((T.cumsum, torch.cumsum(x, -1)), (T.cummax, torch.cummax(x, -1).values),
                   (T.logcumsumexp, torch.logcumsumexp(x, -1))):
        with torch.no_grad():
            got = f(T.from_torch(x.cuda())).data()
        torch.testing.assert_close(got.cpu(), ref, rtol=1e-5, atol=1e-4)
    inf = torch.tensor([[float("-inf"), 1.0, float("-inf"), 2.0]])
    with torch.no_grad():
        got = T.logcumsumexp(T.from_torch(inf.cuda())).data().cpu()
    torch.testing.assert_close(got, torch.logcumsumexp(inf, -1))
