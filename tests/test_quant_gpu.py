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
