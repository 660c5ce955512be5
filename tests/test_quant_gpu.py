"""W4A8 decode kernels against plain fp32 PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,Hq,Hkv,D,cap,length,splits", [
    (1, 4, 1, 128, 776, 700, 0), (2, 8, 2, 128, 300, 300, 3), (3, 4, 4, 64, 130, 1, 4),
    (2, 8, 1, 64, 257, 129, 1), (32, 4, 1, 128, 776, 513, 0), (1, 2, 1, 128, 64, 5, 7)])
def test_decode_attention_split_kv(B, Hq, Hkv, D, cap, length, splits):
    from mimir_b200.ops import quant_cuda as Q
    from mimir_b200.ops._util import check_error_word
    torch.manual_seed(B * 100 + length)
    dev = "cuda"
    q = torch.randn(B, Hq, D, device=dev).bfloat16()
    kc = torch.randn(B, Hkv, cap, D, device=dev).half()
    vc = torch.randn(B, Hkv, cap, D, device=dev).half()
    ln = torch.tensor([length], dtype=torch.int32, device=dev)
    out = Q.attn_decode(q, kc, vc, ln, splits=splits)
    out2 = Q.attn_decode(q, kc, vc, ln, splits=splits)      # the arrival counters reset themselves
    g = Hq // Hkv
    k = kc[:, :, :length].float().repeat_interleave(g, 1)
    v = vc[:, :, :length].float().repeat_interleave(g, 1)
    s = torch.einsum("bhd,bhtd->bht", q.float(), k) * D ** -0.5
    ref = torch.einsum("bht,bhtd->bhd", torch.softmax(s, -1), v)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    assert torch.equal(out, out2)
    assert check_error_word() == 0


@pytest.mark.parametrize("B,N,K,splits", [(1, 768, 4096, 0), (32, 4096, 512, 0), (5, 1000, 1792, 3),
                                          (17, 256, 14336, 0), (32, 3584, 4096, 1), (8, 132, 128, 0)])
def test_q4_tensor_core_product(B, N, K, splits):
    from mimir_b200.ops import quant_cuda as Q
    from mimir_b200.ops.quant import Q4_0, dequantize_raw, quantize_q4_0
    from mimir_b200.ops._util import check_error_word
    torch.manual_seed(B + N)
    dev = "cuda"
    w = torch.randn(N, K) * 0.05
    raw = quantize_q4_0(w)
    wd = dequantize_raw(Q4_0, raw, w.numel()).view(N, K).to(dev)
    wt = Q.TiledQ4.from_planar(Q.PlanarQ4.from_ggml(raw.reshape(-1).to(dev), N, K))
    x = torch.randn(B, K, device=dev).bfloat16()
    res = torch.randn(B, N, device=dev).bfloat16()
    scratch = Q.TcScratch(B * N, dev)
    ref = x.float() @ wd.t()
    out = Q.q4_tc(wt, x, torch.empty(B, N, device=dev), scratch, splits=splits)
    tol = 2e-2 * ref.abs().max().item()
    assert (out - ref).abs().max().item() < tol, ((out - ref).abs().max().item(), tol)
    out2 = Q.q4_tc(wt, x, torch.empty(B, N, device=dev, dtype=torch.bfloat16), scratch, residual=res, splits=splits)
    assert (out2.float() - (ref + res.float())).abs().max().item() < tol + 2e-2 * res.abs().max().item()
    assert check_error_word() == 0


@pytest.mark.parametrize("mode,rows,K", [(0, 3, 512), (1, 2, 4096), (2, 5, 1792), (1, 32, 4096), (2, 1, 14336)])
def test_round_act_q8(mode, rows, K):
    from mimir_b200.ops import quant_cuda as Q
    torch.manual_seed(mode + K)
    x = torch.randn(rows, 2 * K if mode == 2 else K, device="cuda").bfloat16()
    gamma = (1 + 0.1 * torch.randn(K, device="cuda")).bfloat16()
    y = Q.round_act_q8(x, torch.empty(rows, K, device="cuda", dtype=torch.bfloat16), K, mode, gamma)
    xf = x.float()
    if mode == 1:
        t = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).bfloat16().float() * gamma.float()
        t = t.bfloat16().float()
    elif mode == 2:
        t = torch.nn.functional.silu(xf[:, :K]) * xf[:, K:]
    else:
        t = xf
    blocks = t.view(rows, K // 32, 32)
    d = blocks.abs().amax(-1, keepdim=True) / 127
    ref = (torch.round(blocks / d.clamp_min(1e-30)) * d).view(rows, K)
    err = (y.float() - ref).abs().max().item()
    assert err <= 1.01 * d.max().item() + 1e-3, (err, d.max().item())     # at most one quantisation step
    assert (y.float() - ref).abs().mean().item() < 0.02 * ref.abs().mean().item() + 1e-4


def _random_blocks(code, N, K, gen):
    """Random but finite ggml blocks: random payload bytes, small fp16 scales."""
    from mimir_b200.ops import quant as Q
    per, vals = {Q.Q8_0: (34, 32), Q.Q4_0: (18, 32), Q.Q4_K: (144, 256), Q.Q6_K: (210, 256)}[code]
    nb = N * K // vals
    raw = torch.randint(0, 256, (nb, per), dtype=torch.uint8, generator=gen)
    scale = (torch.rand(nb, generator=gen) * 0.02 + 0.001).to(torch.float16).view(torch.uint8).reshape(nb, 2)
    if code in (Q.Q8_0, Q.Q4_0):
        raw[:, 0:2] = scale
    elif code == Q.Q4_K:
        raw[:, 0:2] = scale
        raw[:, 2:4] = (torch.rand(nb, generator=gen) * 0.01).to(torch.float16).view(torch.uint8).reshape(nb, 2)
    else:
        raw[:, 208:210] = scale
    return raw.reshape(-1)


@pytest.mark.gpu
@pytest.mark.parametrize("code_name", ["Q8_0", "Q4_0", "Q4_K", "Q6_K"])
@pytest.mark.parametrize("B,N,K,dtype", [(1, 64, 512, torch.float32), (3, 130, 1024, torch.bfloat16),
                                         (9, 48, 256, torch.float32)])
def test_ggml_block_gemv_reads_the_file_encoding(code_name, B, N, K, dtype):
    """The in-place GEMV over ggml blocks against dequantise (CPU restatement) + fp32 matmul."""
    from mimir_b200.io.mim import QuantizedTensor
    from mimir_b200.ops import quant as Q
    from mimir_b200.ops import quant_cuda as QC
    code = getattr(Q, code_name)
    gen = torch.Generator().manual_seed(B * 1000 + N + K + code)
    raw = _random_blocks(code, N, K, gen)
    w = Q.dequantize_raw(code, raw, N * K).view(N, K)
    x = torch.randn(B, K, generator=gen).to(dtype)
    want = x.float() @ w.t()
    bias = torch.randn(N, generator=gen)
    got = QC.qgemv_ggml(code, raw.cuda(), N, K, x.cuda(), bias=bias.cuda())
    torch.testing.assert_close(got.cpu(), want + bias, rtol=2e-4, atol=2e-3)
    # the lazy layer's quantised product takes the same path for few rows, the GPU dequantiser for many
    qt = QuantizedTensor(code, (N, K), raw.cuda())
    torch.testing.assert_close(Q.qmatmul_t(x.cuda(), qt).float().cpu(), want.to(dtype).float(), rtol=2e-2, atol=2e-2)
    xl = torch.randn(40, K, generator=gen)
    torch.testing.assert_close(Q.qmatmul_t(xl.cuda(), qt).cpu(), xl @ w.t(), rtol=2e-4, atol=2e-3)
