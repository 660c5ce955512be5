"""Native CPU products over ggml blocks against the dequantisation oracle (reference:
backend/cpu/quant_test.go; formats as in tensor/quant.go)."""
import pytest
import torch

from mimir_b200.ops import quant as Q
from mimir_b200.ops import quant_cpu


def _random_blocks(code, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    vals, nbytes = Q.BLOCK[code]
    raw = torch.randint(0, 256, (n * k // vals, nbytes), dtype=torch.uint8, generator=g)
    scale = (torch.rand(raw.shape[0], generator=g) * 0.02 + 0.001).to(torch.float16).view(torch.uint8).reshape(-1, 2)
    if code in (Q.Q8_0, Q.Q4_0):
        raw[:, :2] = scale
    elif code == Q.Q4_K:
        raw[:, 0:2] = scale
        raw[:, 2:4] = (torch.rand(raw.shape[0], generator=g) * 0.01).to(torch.float16).view(torch.uint8).reshape(-1, 2)
    else:
        raw[:, 208:210] = scale
    return raw.reshape(-1)


@pytest.mark.parametrize("code", [Q.Q8_0, Q.Q4_0, Q.Q4_K, Q.Q6_K])
@pytest.mark.parametrize("rows", [1, 3, 8, 11])
def test_exact_product_equals_the_dequantised_product(code, rows):
    n, k = 37, 512
    raw = _random_blocks(code, n, k, code + rows)
    w = Q.dequantize_raw(code, raw, n * k).view(n, k).double()
    x = torch.randn(rows, k)
    want = x.double() @ w.t()
    got = quant_cpu.qgemv(code, raw, n, k, x, "exact")
    assert got.shape == (rows, n)
    assert torch.allclose(got.double(), want, rtol=1e-5, atol=1e-5 * float(want.abs().max()))


@pytest.mark.parametrize("code", [Q.Q8_0, Q.Q4_0, Q.Q4_K, Q.Q6_K])
def test_int8_product_stays_within_the_rounding_of_the_activations(code):
    if not quant_cpu.has_int8():
        pytest.skip("this CPU has no AVX-512 VNNI")
    n, k = 64, 1024
    raw = _random_blocks(code, n, k, 7 * code)
    w = Q.dequantize_raw(code, raw, n * k).view(n, k).double()
    x = torch.randn(5, k)
    want = x.double() @ w.t()
    got = quant_cpu.qgemv(code, raw, n, k, x, "int8").double()
    # the oracle of the int8 path: the same product with the activations rounded to int8 blocks
    group = 256 if code in (Q.Q4_K, Q.Q6_K) else 32            # the K-quants share one activation scale per super-block
    xb = x.reshape(5, k // group, group)
    d = xb.abs().amax(-1, keepdim=True) / 127
    xq = (torch.round(xb / d.clamp_min(1e-30)) * d).reshape(5, k).double()
    rounded = xq @ w.t()
    assert torch.allclose(got, rounded, rtol=1e-4, atol=1e-4 * float(want.abs().max()))
    assert float((got - want).abs().max()) < 2e-2 * float(want.abs().max())


def test_threads_row_split_and_bad_arguments():
    code, n, k = Q.Q4_K, 203, 512                       # a row count no thread count divides
    raw = _random_blocks(code, n, k, 5)
    x = torch.randn(2, k)
    ref = quant_cpu.qgemv(code, raw, n, k, x, "exact")
    old = quant_cpu.set_threads(3)
    try:
        assert torch.equal(quant_cpu.qgemv(code, raw, n, k, x, "exact"), ref)
        quant_cpu.set_threads(1)
        assert torch.equal(quant_cpu.qgemv(code, raw, n, k, x, "exact"), ref)
    finally:
        quant_cpu.set_threads(old)
    with pytest.raises(ValueError):
        quant_cpu.qgemv(code, raw, n, 500, torch.randn(1, 500), "exact")       # K not a multiple of the block
    with pytest.raises(ValueError):
        quant_cpu.qgemv(code, raw, n, k, torch.randn(1, k + 256), "exact")


def test_lazy_qmatmul_takes_the_native_path_for_few_rows_on_the_cpu():
    import mimir_b200.tensor as T
    from mimir_b200.io import mim
    n, k = 48, 256
    raw = _random_blocks(Q.Q6_K, n, k, 9)
    qt = mim.QuantizedTensor(Q.Q6_K, (n, k), raw)
    x = torch.randn(2, 3, k)
    want = x @ Q.dequantize(qt).t()
    got = T.matmul_t(T.tensor(x), qt).data()
    assert got.shape == (2, 3, n) and torch.allclose(got, want, rtol=1e-4, atol=1e-4 * float(want.abs().max()))
