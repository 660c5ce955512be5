"""MNIST-shaped CNN on the native conv / pool / GEMM kernels against fp32 PyTorch: 10-step loss curve."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_mnist_cnn_ten_step_loss_curve_matches_pytorch():
    from mimir_b200.models.cnn import MnistCNN, reference
    from mimir_b200.ops._util import check_error_word
    torch.manual_seed(0)
    N = 128
    eng = MnistCNN(N, "cuda", seed=1, lr=1e-3, weight_decay=0.01)
    ref = reference({k: v.cpu() for k, v in eng.state().items()}, "cuda")
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=0.01)
    xs = torch.randn(10, N, 1, 28, 28, device="cuda")
    ys = torch.randint(0, 10, (10, N), device="cuda")
    # a learnable signal: the label shifts the mean of the image
    xs = xs + ys.view(10, N, 1, 1, 1).float() * 0.2
    ours, theirs = [], []
    for i in range(10):
        ours.append(eng.train_step(xs[i], ys[i]).item())
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(ref(xs[i]), ys[i])
        loss.backward()
        opt.step()
        theirs.append(loss.item())
    assert check_error_word() == 0
    assert eng.launches_per_step > 15
    for a, b in zip(ours, theirs):
        assert abs(a - b) < 0.03 * max(1.0, abs(b)), (ours, theirs)
    assert ours[-1] < ours[0]
