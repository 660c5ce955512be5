"""The shared case table (``mimir_b200/utils/conformance.py``) on the GPU in float32 against the
float64 oracle files, the way the reference runs the same kerneltest cases on every backend
(backend/internal/kerneltest/kerneltest.go:58-120, backend/cuda/kernel_test.go:62-80)."""
import pytest
import torch

from mimir_b200.utils import conformance as conf

# float32 attention goes through PyTorch's fused kernels, whose tensor-core precision mode differs
# between builds, and the running sums take the native scan kernel outside autograd: both have
# their own GPU tests with their own tolerances
ELSEWHERE = {"attention_causal", "attention_gqa_cross", "cumsum_axis1", "unary_lgamma"}


@pytest.mark.gpu
def test_gpu_float32_is_conformant(tmp_path):
    import mimir_b200.tensor as T
    golden = str(tmp_path / "golden")
    conf.generate(golden)
    only = {c.name for c in conf.CASES} - ELSEWHERE
    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False                 # float32 convolutions in full precision, like the oracle
    try:
        assert conf.check(golden, device=T.GPU(0), only=only) == []
    finally:
        torch.backends.cudnn.allow_tf32 = old
