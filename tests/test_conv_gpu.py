"""Implicit-GEMM convolution and pooling kernels against fp32 PyTorch."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

CASES = [  # N, Ci, Co, H, W, K, pad, dil, relu
    (4, 1, 32, 28, 28, 3, 1, 1, True),
    (3, 32, 64, 14, 14, 3, 1, 1, True),
    (2, 64, 128, 17, 23, 3, 1, 1, False),
    (2, 96, 40, 9, 40, 5, 2, 1, False),
    (1, 128, 256, 32, 32, 1, 0, 1, False),
    (2, 64, 64, 20, 20, 3, 2, 2, False),
    (2, 16, 16, 12, 12, 3, 0, 1, False),
]


@pytest.mark.parametrize("N,Ci,Co,H,W,K,pad,dil,relu", CASES)
def test_conv2d_fwd_dgrad_wgrad(N, Ci, Co, H, W, K, pad, dil, relu):
    from mimir_b200.ops import conv as C
    from mimir_b200.ops._util import check_error_word
    torch.manual_seed(N * 7 + Ci + Co)
    dev = "cuda"
    x = torch.randn(N, Ci, H, W, device=dev).bfloat16().float()
    w = (torch.randn(Co, Ci, K, K, device=dev) / (Ci * K * K) ** 0.5).bfloat16().float()
    b = torch.randn(Co, device=dev)
    ref = F.conv2d(x, w, b, padding=pad, dilation=dil)
    if relu:
        ref = ref.relu()
    xn = C.to_nhwc(x)
    bias = torch.zeros(C.pad64(Co), device=dev)
    bias[:Co] = b
    y = C.conv2d_fwd(xn, C.pack_filter(w), K, K, pad, dil, bias=bias, relu=relu)
    got = C.from_nhwc(y, Co).float()
    assert got.shape == ref.shape
    assert torch.allclose(got, ref, atol=3e-2, rtol=3e-2), (got - ref).abs().max()
    assert y[..., Co:].abs().max() == 0 if y.shape[-1] > Co else True

    dy = torch.randn_like(ref).bfloat16().float()
    dyn = C.to_nhwc(dy)
    dx_ref = torch.nn.grad.conv2d_input(x.shape, w, dy, padding=pad, dilation=dil)
    dw_ref = torch.nn.grad.conv2d_weight(x, w.shape, dy, padding=pad, dilation=dil)
    dx = C.from_nhwc(C.conv2d_dgrad(dyn, C.pack_filter_dgrad(w), K, K, pad, dil), Ci).float()
    assert torch.allclose(dx, dx_ref, atol=4e-2, rtol=3e-2), (dx - dx_ref).abs().max()
    dw = C.unpack_filter_grad(C.conv2d_wgrad(dyn, xn, Co, K, K, pad, dil), w.shape)
    scale = dw_ref.abs().max().item()
    assert (dw - dw_ref).abs().max().item() < 2e-2 * scale + 1e-3, ((dw - dw_ref).abs().max().item(), scale)
    # accumulate adds to what is there; a forced split count gives the same sums
    dw2 = C.conv2d_wgrad(dyn, xn, Co, K, K, pad, dil, out=C.conv2d_wgrad(dyn, xn, Co, K, K, pad, dil, splits=3),
                         accumulate=True, splits=1)
    assert torch.allclose(C.unpack_filter_grad(dw2, w.shape), 2 * dw, atol=2e-2 * scale + 1e-3)
    assert check_error_word() == 0


@pytest.mark.parametrize("N,C_,H,W,k,s", [(4, 64, 28, 28, 2, 2), (2, 128, 15, 17, 3, 2), (1, 64, 9, 9, 3, 1)])
def test_maxpool_fwd_bwd(N, C_, H, W, k, s):
    from mimir_b200.ops import conv as C
    torch.manual_seed(3)
    x = torch.randn(N, C_, H, W, device="cuda").bfloat16().float().requires_grad_(True)
    ref = F.max_pool2d(x, k, s)
    dy = torch.randn_like(ref).bfloat16().float()
    ref.backward(dy)
    xn = C.to_nhwc(x.detach())
    y, arg = C.maxpool2d_fwd(xn, k, s)
    assert torch.equal(C.from_nhwc(y, C_).float(), ref.detach())
    dx = C.maxpool2d_bwd(C.to_nhwc(dy), arg, xn.shape, k, s)
    assert torch.allclose(C.from_nhwc(dx, C_).float(), x.grad, atol=2e-2, rtol=2e-2)


def test_relu_bwd():
    from mimir_b200.ops import conv as C
    y = torch.randn(4096, device="cuda").bfloat16()
    dy = torch.randn(4096, device="cuda").bfloat16()
    assert torch.equal(C.relu_bwd(y, dy), torch.where(y > 0, dy, torch.zeros_like(dy)))
