"""MNIST-shaped CNN trained on the native sm_100a kernels (reference model:
examples/mnist/main.go:97-101 — conv 1->32 3x3 pad 1, ReLU, max-pool 2, conv 32->64 3x3 pad 1,
ReLU, max-pool 2, flatten, linear 3136->128, ReLU, linear 128->10; AdamW).

Activations are bf16 NHWC with channels padded to 64; the convolutions are implicit GEMMs on the
tensor cores (forward with bias + ReLU in the epilogue, input gradient as the same kernel on the
flipped filter, weight gradient as a split contraction over pixel patches), pooling keeps a
byte argmax, the linear layers use the GEMM kernel, the loss is the fused cross-entropy row
kernel, and one AdamW launch updates the flat fp32 master parameters and their bf16 copies.
Parameters keep PyTorch's shapes and flatten order, so ``load_torch`` / ``reference`` can compare
the engine with a plain fp32 PyTorch model step by step.
"""
from __future__ import annotations

import math

import torch

from ..ops import conv as C
from ..ops import kernels as K
from ..ops.gemm import gemm

SHAPES = [("c1w", (32, 1, 3, 3)), ("c1b", (32,)), ("c2w", (64, 32, 3, 3)), ("c2b", (64,)),
          ("f1w", (128, 64 * 7 * 7)), ("f1b", (128,)), ("f2w", (10, 128)), ("f2b", (10,))]


class MnistCNN:
    def __init__(self, batch: int, device="cuda", seed: int = 0, lr: float = 1e-3, weight_decay: float = 0.01,
                 betas=(0.9, 0.999), eps: float = 1e-8):
        self.N, self.dev = batch, torch.device(device)
        self.lr, self.wd, self.betas, self.eps, self.t = lr, weight_decay, betas, eps, 0
        n = sum(math.prod(s) for _, s in SHAPES)
        n = (n + 7) // 8 * 8
        f32 = dict(dtype=torch.float32, device=self.dev)
        self.master, self.grad = torch.zeros(n, **f32), torch.zeros(n, **f32)
        self.m, self.v = torch.zeros(n, **f32), torch.zeros(n, **f32)
        self.param = torch.zeros(n, dtype=torch.bfloat16, device=self.dev)
        self.views, self.gviews, self.pviews, off = {}, {}, {}, 0
        g = torch.Generator(device="cpu").manual_seed(seed)
        for name, shape in SHAPES:
            k = math.prod(shape)
            self.views[name] = self.master[off: off + k].view(shape)
            self.gviews[name] = self.grad[off: off + k].view(shape)
            self.pviews[name] = self.param[off: off + k].view(shape)
            fan_in = math.prod(shape[1:]) if len(shape) > 1 else None
            if fan_in:  # PyTorch's default: uniform(-1/sqrt(fan_in), 1/sqrt(fan_in)) for weight and bias
                bound = 1 / math.sqrt(fan_in)
                self.views[name].copy_((torch.rand(shape, generator=g) * 2 - 1) * bound)
                self._last_bound = bound
            else:
                self.views[name].copy_((torch.rand(shape, generator=g) * 2 - 1) * self._last_bound)
            off += k
        self.param.copy_(self.master)
        self.loss_rows = torch.zeros(batch, **f32)
        self.loss = torch.zeros(1, **f32)
        self.colsum_scratch = torch.zeros(64 * 16384, **f32)
        self.launches_per_step = 0

    # ------------------------------------------------------------------ io
    def load_torch(self, state: dict) -> None:
        for name, _ in SHAPES:
            self.views[name].copy_(state[name].to(self.dev))
        self.param.copy_(self.master)

    def state(self) -> dict:
        return {k: v.clone() for k, v in self.views.items()}

    # ------------------------------------------------------------- forward
    def _packed(self):
        p, dev = self.pviews, self.dev
        b1 = torch.zeros(64, device=dev); b1[:32] = p["c1b"].float()
        b2 = p["c2b"].float().contiguous()
        # fc1 reads the pooled map in (h, w, c) order: reorder PyTorch's (c, h, w) columns
        f1 = p["f1w"].view(128, 64, 7, 7).permute(0, 2, 3, 1).reshape(128, 3136).contiguous()
        f2 = torch.zeros(16, 128, dtype=torch.bfloat16, device=dev); f2[:10] = p["f2w"]
        fb2 = torch.zeros(16, dtype=torch.bfloat16, device=dev); fb2[:10] = p["f2b"]
        return dict(c1=C.pack_filter(p["c1w"]), c2=C.pack_filter(p["c2w"]), c2d=C.pack_filter_dgrad(p["c2w"]),
                    b1=b1, b2=b2, f1=f1, f1b=p["f1b"].contiguous(), f2=f2, f2b=fb2)

    def forward(self, x: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """x [N, 1, 28, 28] (any float dtype, on the device), targets int64 [N]; returns the mean loss (device scalar)."""
        N = self.N
        w = self.w = self._packed()
        a = self.act = {}
        a["x"] = C.to_nhwc(x)
        a["y1"] = C.conv2d_fwd(a["x"], w["c1"], 3, 3, 1, bias=w["b1"], relu=True)
        a["p1"], a["i1"] = C.maxpool2d_fwd(a["y1"], 2)
        a["y2"] = C.conv2d_fwd(a["p1"], w["c2"], 3, 3, 1, bias=w["b2"], relu=True)
        a["p2"], a["i2"] = C.maxpool2d_fwd(a["y2"], 2)
        flat = a["p2"].view(N, 3136)
        a["z1"] = gemm(flat, w["f1"], bias=w["f1b"])
        a["a1"] = K.act_fwd(a["z1"], torch.empty_like(a["z1"]), "relu")
        a["logits"] = gemm(a["a1"], w["f2"], bias=w["f2b"])
        self.targets = targets
        K.cross_entropy(a["logits"], targets, self.loss_rows, a["logits"], self.loss, 10, 1.0 / N, 1.0 / N)
        return self.loss

    # ------------------------------------------------------------ backward
    def backward(self) -> None:
        """Gradients of the mean loss into ``self.grad`` (the cross-entropy kernel already left
        dlogits in place of the logits)."""
        N, a, w, g = self.N, self.act, self.w, self.gviews
        dlog = a["logits"]                                    # [N, 16] bf16, columns >= 10 are zero
        dlog[:, 10:].zero_()
        dw2 = gemm(dlog, a["a1"], a_mn=True, b_mn=True, out_dtype=torch.float32)      # [16, 128]
        g["f2w"].copy_(dw2[:10])
        g["f2b"].copy_(K.colsum(dlog, torch.empty(16, device=self.dev), self.colsum_scratch)[:10])
        da1 = gemm(dlog, w["f2"], b_mn=True)                                           # [N, 128]
        dz1 = K.act_bwd(a["z1"], da1, torch.empty_like(da1), "relu")
        dw1 = gemm(dz1, a["p2"].view(N, 3136), a_mn=True, b_mn=True, out_dtype=torch.float32)  # [128, 3136] (h, w, c)
        g["f1w"].copy_(dw1.view(128, 7, 7, 64).permute(0, 3, 1, 2).reshape(128, 3136))
        g["f1b"].copy_(K.colsum(dz1, torch.empty(128, device=self.dev), self.colsum_scratch))
        dp2 = gemm(dz1, w["f1"], b_mn=True).view(N, 7, 7, 64)
        dy2 = C.relu_bwd(a["y2"], C.maxpool2d_bwd(dp2, a["i2"], a["y2"].shape, 2))
        g["c2w"].copy_(C.unpack_filter_grad(C.conv2d_wgrad(dy2, a["p1"], 64, 3, 3, 1), (64, 32, 3, 3)))
        g["c2b"].copy_(K.colsum(dy2.view(-1, 64), torch.empty(64, device=self.dev), self.colsum_scratch))
        dp1 = C.conv2d_dgrad(dy2, w["c2d"], 3, 3, 1)
        dy1 = C.relu_bwd(a["y1"], C.maxpool2d_bwd(dp1, a["i1"], a["y1"].shape, 2))
        g["c1w"].copy_(C.unpack_filter_grad(C.conv2d_wgrad(dy1, a["x"], 32, 3, 3, 1), (32, 1, 3, 3)))
        g["c1b"].copy_(K.colsum(dy1.view(-1, 64), torch.empty(64, device=self.dev), self.colsum_scratch)[:32])

    def step(self) -> None:
        self.t += 1
        K.adamw_flat(self.master, self.param, self.grad, self.m, self.v, lr=self.lr, beta1=self.betas[0],
                     beta2=self.betas[1], eps=self.eps, wd=self.wd, step=self.t)

    def train_step(self, x, targets) -> torch.Tensor:
        from .. import _native
        before = _native.lib().mimir_launch_count()
        loss = self.forward(x, targets)
        self.backward()
        self.step()
        self.launches_per_step = _native.lib().mimir_launch_count() - before
        return loss


def reference(state: dict | None = None, device="cpu") -> torch.nn.Module:
    """The same network in plain fp32 PyTorch (optionally with the engine's parameters)."""
    nn = torch.nn
    net = nn.Sequential(nn.Conv2d(1, 32, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2), nn.Conv2d(32, 64, 3, padding=1),
                        nn.ReLU(), nn.MaxPool2d(2), nn.Flatten(), nn.Linear(3136, 128), nn.ReLU(), nn.Linear(128, 10))
    if state is not None:
        with torch.no_grad():
            for mod, wn, bn in ((net[0], "c1w", "c1b"), (net[3], "c2w", "c2b"), (net[7], "f1w", "f1b"), (net[9], "f2w", "f2b")):
                mod.weight.copy_(state[wn])
                mod.bias.copy_(state[bn])
    return net.to(device)
