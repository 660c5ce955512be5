"""tcgen05 GEMM against a plain fp32 PyTorch product of the same bf16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    return A @ B


def _check(out, ref, K):
    """bf16 output: within 2e-2 of the largest element overall AND, row by row, within 2e-2 of that
    row's own largest element (an error confined to one tile edge or one group of rows shows)."""
    diff = (out.float() - ref).abs()
    scale = ref.abs().max().item() + 1e-6
    assert diff.max().item() / scale < 2e-2, f"max err {diff.max().item()} vs scale {scale}"
    row_scale = ref.abs().amax(dim=1) + 1e-3 * scale
    worst = (diff.amax(dim=1) / row_scale).max().item()
    assert worst < 2e-2, f"worst row error {worst}"
    col_scale = ref.abs().amax(dim=0) + 1e-3 * scale
    assert (diff.amax(dim=0) / col_scale).max().item() < 2e-2


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (1000, 776, 136), (4096, 768, 768), (130, 264, 1024)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_fp32_output_is_exact_to_rounding(M, N, K, a_mn, b_mn):
    """With fp32 output only the accumulation order differs from the reference product: 1e-3 of the
    row's largest element, per row."""
    from mimir_b200.ops import gemm
    from mimir_b200.ops._util import check_error_word
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a 16-byte row pitch")
    torch.manual_seed(M + N + K)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert check_error_word() == 0 and out.dtype == torch.float32
    ref = _ref(a, b, a_mn, b_mn)
    diff = (out - ref).abs()
    row_scale = ref.abs().amax(dim=1) + 1e-6
    assert (diff.amax(dim=1) / row_scale).max().item() < 1e-3


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K,bn", [
    (128, 128, 64, 128), (256, 256, 128, 256), (384, 512, 320, 0), (1000, 776, 136, 0),
    (4096, 768, 768, 0), (200, 64, 72, 64), (130, 264, 1024, 128),
])
def test_gemm_layouts(M, N, K, bn, a_mn, b_mn):
    from mimir_b200.ops import gemm
    from mimir_b200.ops._util import check_error_word
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a 16-byte row pitch")
    torch.manual_seed(M * 7 + N * 3 + K)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
    assert check_error_word() == 0
    _check(out, _ref(a, b, a_mn, b_mn), K)


def test_gemm_epilogues():
    from mimir_b200.ops import gemm
    from mimir_b200.ops._util import check_error_word
    torch.manual_seed(1)
    M, N, K = 512, 384, 256
    a = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    z = a.float() @ w.float().t() + bias.float()
    pre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, w, bias=bias, gelu=True, aux_out=pre)
    _check(pre, z, K)
    _check(out, torch.nn.functional.gelu(z, approximate="tanh"), K)
    out = gemm(a, w, bias=bias, residual=True, aux=res)
    _check(out, z + res.float(), K)
    # d/dz gelu(z) via autograd
    zz = res.float().clone().requires_grad_(True)
    torch.nn.functional.gelu(zz, approximate="tanh").sum().backward()
    out = gemm(a, w, mul_dgelu=True, aux=res)
    _check(out, (a.float() @ w.float().t()) * zz.grad, K)
    out32 = torch.ones(M, N, device="cuda")
    gemm(a, w, out=out32, accumulate=True, alpha=0.5)
    _check(out32, 1 + 0.5 * (a.float() @ w.float().t()), K)
    assert check_error_word() == 0


@pytest.mark.parametrize("splits", [2, 4, 7])
def test_gemm_split_k(splits):
    from mimir_b200.ops import gemm
    from mimir_b200.ops._util import check_error_word
    torch.manual_seed(2)
    M, N, K = 256, 256, 2048
    a = torch.randn(K, M, device="cuda").bfloat16()
    b = torch.randn(K, N, device="cuda").bfloat16()
    out = gemm(a, b, a_mn=True, b_mn=True, splits=splits)
    assert check_error_word() == 0
    _check(out, _ref(a, b, True, True), K)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K,bn", [
    (256, 256, 64, 1256), (512, 384, 192, 1128), (1000, 776, 136, 1256), (4096, 768, 768, 1256),
    (392, 520, 72, 1128), (2048, 2304, 768, 1256),
])
def test_gemm_cta_pair_layouts(M, N, K, bn, a_mn, b_mn):
    """The cta_group::2 kernel (forced with bn + 1000) against the fp32 product."""
    from mimir_b200.ops import gemm
    from mimir_b200.ops._util import check_error_word
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a 16-byte row pitch")
    torch.manual_seed(M + N + K)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
    assert check_error_word() == 0
    _check(out, _ref(a, b, a_mn, b_mn), K)


def test_gemm_cta_pair_split_k_and_epilogue():
    from mimir_b200.ops import gemm
    from mimir_b200.ops._util import check_error_word
    torch.manual_seed(5)
    M, N, K = 512, 256, 2048
    a = torch.randn(K, M, device="cuda").bfloat16()
    b = torch.randn(K, N, device="cuda").bfloat16()
    out = gemm(a, b, a_mn=True, b_mn=True, splits=4, bn=1256)
    _check(out, _ref(a, b, True, True), K)
    x = torch.randn(M, 256, device="cuda").bfloat16()
    w = (torch.randn(N, 256, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    out = gemm(x, w, bias=bias, residual=True, aux=res, bn=1128)
    _check(out, x.float() @ w.float().t() + bias.float() + res.float(), 256)
    assert check_error_word() == 0


@pytest.mark.parametrize("bn", [1256, 1128])
def test_gemm_cta_pair_tma_store_epilogues(bn):
    """bf16 outputs of the pair kernel leave through TMA stores, with every fused epilogue."""
    from mimir_b200.ops import gemm
    from mimir_b200.ops._util import check_error_word
    torch.manual_seed(9)
    M, N, K = 1000, 712, 256  # ragged in both directions
    a = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    z = a.float() @ w.float().t() + bias.float()
    pre = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, w, bias=bias, gelu=True, aux_out=pre, bn=bn)
    _check(pre, z, K)
    _check(out, torch.nn.functional.gelu(z, approximate="tanh"), K)
    out = gemm(a, w, bias=bias, residual=True, aux=res, bn=bn)
    _check(out, z + res.float(), K)
    zz = res.float().clone().requires_grad_(True)
    torch.nn.functional.gelu(zz, approximate="tanh").sum().backward()
    out = gemm(a, w, mul_dgelu=True, aux=res, bn=bn)
    _check(out, (a.float() @ w.float().t()) * zz.grad, K)
    # a strided output (columns of a wider matrix) must leave its neighbours alone
    wide = torch.full((M, 2 * N), 3.0, device="cuda", dtype=torch.bfloat16)
    gemm(a, w, out=wide[:, :N], bn=bn)
    _check(wide[:, :N], a.float() @ w.float().t(), K)
    assert (wide[:, N:] == 3.0).all()
    assert check_error_word() == 0
