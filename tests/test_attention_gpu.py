"""tcgen05 attention forward / backward against fp32 PyTorch on the same bf16 inputs."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, causal, offset):
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    if causal:
        i = torch.arange(Tq, device=q.device)[:, None]
        j = torch.arange(Tk, device=q.device)[None]
        s = s.masked_fill(j > i + offset, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.softmax(s, -1) @ vf
    return o.permute(0, 2, 1, 3), lse


CASES = [
    # B, Tq, Tk, Hq, Hkv, D, causal
    (2, 128, 128, 2, 2, 64, True),
    (1, 256, 256, 4, 2, 64, True),
    (2, 200, 200, 2, 1, 64, True),
    (1, 384, 384, 2, 2, 128, True),
    (1, 128, 320, 2, 2, 64, True),
    (1, 160, 160, 2, 2, 64, False),
    (1, 100, 228, 4, 1, 128, False),
    (2, 1024, 1024, 3, 3, 64, True),
]


@pytest.mark.parametrize("B,Tq,Tk,Hq,Hkv,D,causal", CASES)
def test_attention_fwd_bwd(B, Tq, Tk, Hq, Hkv, D, causal):
    from mimir_b200.ops.attention import attention_bwd, attention_fwd
    from mimir_b200.ops._util import check_error_word
    torch.manual_seed(B * 1000 + Tq + Tk + D)
    q = torch.randn(B, Tq, Hq, D, device="cuda").bfloat16().requires_grad_(True)
    k = torch.randn(B, Tk, Hkv, D, device="cuda").bfloat16().requires_grad_(True)
    v = torch.randn(B, Tk, Hkv, D, device="cuda").bfloat16().requires_grad_(True)
    do = torch.randn(B, Tq, Hq, D, device="cuda").bfloat16()
    offset = Tk - Tq
    o_ref, lse_ref = _ref(q, k, v, causal, offset)
    o_ref.backward(do.float())
    out = torch.empty(B, Tq, Hq, D, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(B, Hq, Tq, device="cuda")
    attention_fwd(q.detach(), k.detach(), v.detach(), out, lse, causal=causal)
    assert check_error_word() == 0
    assert (out.float() - o_ref).abs().max().item() < 3e-2
    assert (lse - lse_ref).abs().max().item() < 2e-2
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    dsum = torch.empty(B, Hq, Tq, device="cuda")
    attention_bwd(q.detach(), k.detach(), v.detach(), out, do, lse, dsum, dq, dk, dv, causal=causal)
    assert check_error_word() == 0
    for got, ref, name in ((dq, q.grad, "dq"), (dk, k.grad, "dk"), (dv, v.grad, "dv")):
        err = (got.float() - ref.float()).abs().max().item()
        scale = ref.float().abs().max().item()
        assert err < 3e-2 * scale + 2e-2, f"{name}: err {err} scale {scale}"
