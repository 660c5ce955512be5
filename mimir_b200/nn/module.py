"""Module tree, parameter discovery and the basic layers.

Parameters are found by walking attributes (the reference reflects over struct
fields, nn/nn.go:74-153); names follow the attribute path, list elements by
index (``layers.0.weight``).  Initialisation matches the PyTorch defaults the
reference uses (nn/layers.go:36-47); seeds derive from one module seed through
splitmix64 so that a model is reproducible on every device (nn/nn.go:252-268).
"""
from __future__ import annotations

import math

import torch

from .. import tensor as T
from ..tensor.autograd import Buffer, Param
from ..tensor.random import philox_normal, philox_uniform, splitmix64

_seed_state = [0x5EED]


def manual_seed(seed: int) -> None:
    _seed_state[0] = seed


def _next_seed() -> int:
    _seed_state[0] = splitmix64(_seed_state[0])
    return _seed_state[0]


def uniform_init(shape, bound: float, dtype=torch.float32) -> torch.Tensor:
    return ((philox_uniform(shape, _next_seed(), "cpu") * 2 - 1) * bound).to(dtype)


def normal_init(shape, std: float, dtype=torch.float32) -> torch.Tensor:
    return (philox_normal(shape, _next_seed(), "cpu") * std).to(dtype)


class Module:
    """Base class: ``forward`` builds the lazy graph; calling the module calls it."""

    training = True

    def forward(self, *a, **k):
        raise NotImplementedError

    def __call__(self, *a, **k):
        return self.forward(*a, **k)

    # -- discovery
    def named_children(self):
        for name, v in vars(self).items():
            if name.startswith("_nn_skip"):
                continue
            if isinstance(v, Module):
                yield name, v
            elif isinstance(v, (list, tuple)):
                for i, e in enumerate(v):
                    if isinstance(e, Module):
                        yield f"{name}.{i}", e
            elif isinstance(v, dict):
                for k, e in v.items():
                    if isinstance(e, Module):
                        yield f"{name}.{k}", e

    def named_params(self, prefix: str = "", buffers: bool = True):
        for name, v in vars(self).items():
            if isinstance(v, Param) and (buffers or not isinstance(v, Buffer)):
                yield prefix + name, v
            elif isinstance(v, (list, tuple)):
                for i, e in enumerate(v):
                    if isinstance(e, Param) and (buffers or not isinstance(e, Buffer)):
                        yield f"{prefix}{name}.{i}", e
        for cname, child in self.named_children():
            yield from child.named_params(prefix + cname + ".", buffers)

    def parameters(self):
        return [p for _, p in self.named_params(buffers=False)]

    def modules(self):
        yield self
        for _, c in self.named_children():
            yield from c.modules()

    # -- state
    def train(self, mode: bool = True):
        for m in self.modules():
            m.training = mode
        return self

    def eval(self):
        return self.train(False)

    def to(self, device):
        for _, p in self.named_params():
            p.to(device)
        return self

    def cast(self, dtype):
        """Casts floating-point parameters (nn.Cast, nn/dtype.go:32)."""
        for _, p in self.named_params():
            if p.dtype.is_floating_point:
                p.cast(dtype)
        return self

    def zero_grad(self):
        for p in self.parameters():
            p.zero_grad()

    def state_dict(self) -> dict:
        return {n: p._data for n, p in self.named_params()}

    def load_state_dict(self, sd: dict, strict: bool = True):
        have = dict(self.named_params())
        for n, p in have.items():
            if n in sd:
                v = sd[n]
                v = v.dequantize() if hasattr(v, "dequantize") else v
                p.set(v.to(p.dtype))
            elif strict:
                raise KeyError(f"missing tensor {n!r}")
        return self

    def batch_norms(self):
        return [m for m in self.modules() if isinstance(m, _BatchNorm)]


class Sequential(Module):
    def __init__(self, *layers):
        self.layers = list(layers)

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return x


class Linear(Module):
    """``y = x W^T + b`` with ``W`` stored ``[out, in]``; ``W`` may be quantized (nn/layers.go:49-55)."""

    def __init__(self, fan_in: int, fan_out: int, bias: bool = True, dtype=torch.float32):
        bound = 1.0 / math.sqrt(fan_in)
        self.weight = Param(uniform_init((fan_out, fan_in), bound, dtype), "weight")
        self.bias = Param(uniform_init((fan_out,), bound, dtype), "bias") if bias else None
        self.qweight = None  # set to a QuantizedTensor to run on quantized weights

    def forward(self, x):
        if self.qweight is not None:
            y = T.matmul_t(x, self.qweight)
            return y + self.bias.value() if self.bias is not None else y
        return T.matmul_t(x, self.weight.value(), self.bias.value() if self.bias is not None else None)


class _ConvNd(Module):
    _fn = None
    _nd = 2

    def __init__(self, cin, cout, kernel, stride=1, padding=0, dilation=1, groups=1, bias=True, dtype=torch.float32):
        k = (kernel,) * self._nd if isinstance(kernel, int) else tuple(kernel)
        fan_in = cin // groups * math.prod(k)
        bound = 1.0 / math.sqrt(fan_in)
        self.weight = Param(uniform_init((cout, cin // groups, *k), bound, dtype), "weight")
        self.bias = Param(uniform_init((cout,), bound, dtype), "bias") if bias else None
        self.stride, self.padding, self.dilation, self.groups = stride, padding, dilation, groups

    def forward(self, x):
        return type(self)._fn(x, self.weight.value(), self.bias.value() if self.bias is not None else None,
                              self.stride, self.padding, self.dilation, self.groups)


class Conv1d(_ConvNd):
    _fn, _nd = staticmethod(T.conv1d), 1


class Conv2d(_ConvNd):
    _fn, _nd = staticmethod(T.conv2d), 2


class Conv3d(_ConvNd):
    _fn, _nd = staticmethod(T.conv3d), 3


class DepthwiseConv2d(Conv2d):
    def __init__(self, channels, kernel, stride=1, padding=0, bias=True, dtype=torch.float32):
        super().__init__(channels, channels, kernel, stride, padding, 1, channels, bias, dtype)


class _ConvTransposeNd(Module):
    _fn, _nd = None, 2

    def __init__(self, cin, cout, kernel, stride=1, padding=0, output_padding=0, bias=True, dtype=torch.float32):
        k = (kernel,) * self._nd if isinstance(kernel, int) else tuple(kernel)
        bound = 1.0 / math.sqrt(cout * math.prod(k))
        self.weight = Param(uniform_init((cin, cout, *k), bound, dtype), "weight")
        self.bias = Param(uniform_init((cout,), bound, dtype), "bias") if bias else None
        self.stride, self.padding, self.output_padding = stride, padding, output_padding

    def forward(self, x):
        return type(self)._fn(x, self.weight.value(), self.bias.value() if self.bias is not None else None,
                              self.stride, self.padding, self.output_padding)


class ConvTranspose1d(_ConvTransposeNd):
    _fn, _nd = staticmethod(T.conv_transpose1d), 1


class ConvTranspose2d(_ConvTransposeNd):
    _fn, _nd = staticmethod(T.conv_transpose2d), 2


class Embedding(Module):
    def __init__(self, vocab: int, dim: int, dtype=torch.float32):
        self.weight = Param(normal_init((vocab, dim), 1.0, dtype), "weight")

    def forward(self, idx):
        return T.gather_rows(self.weight.value(), idx)


class LayerNorm(Module):
    def __init__(self, dim: int, eps: float = 1e-5, dtype=torch.float32):
        self.weight = Param(torch.ones(dim, dtype=dtype), "weight")
        self.bias = Param(torch.zeros(dim, dtype=dtype), "bias")
        self.eps, self.dim = eps, dim

    def forward(self, x):
        return T.layer_norm(x, self.weight.value(), self.bias.value(), self.eps)


class RMSNorm(Module):
    """Normalises in fp32, rounds to the input dtype, then scales (nn/transformer.go:28-61).  Without
    an ``eps`` it is float32's machine epsilon (2^-23), the reference's and PyTorch's default; Llama
    models pass 1e-5 or 1e-6."""

    def __init__(self, dim: int, eps: float | None = None, dtype=torch.float32):
        self.weight = Param(torch.ones(dim, dtype=dtype), "weight")
        self.eps = 2.0 ** -23 if eps is None else eps

    def forward(self, x):
        return T.rms_norm(x, self.weight.value(), self.eps)


class GroupNorm(Module):
    def __init__(self, groups: int, channels: int, eps: float = 1e-5, dtype=torch.float32):
        self.weight = Param(torch.ones(channels, dtype=dtype), "weight")
        self.bias = Param(torch.zeros(channels, dtype=dtype), "bias")
        self.groups, self.eps = groups, eps

    def forward(self, x):
        """Mean and variance over each group of channels (and all positions) of each example, in tensor ops:
        ``[N, C, ...] -> [N, groups, -1]``, normalised over the last axis, back, then scaled per channel."""
        shape = tuple(x.shape)
        n, c = shape[0], shape[1]
        if c % self.groups:
            return T.core._error_tensor(T.ErrShape(f"group norm of {c} channels in {self.groups} groups"))
        g = T.reshape(x, (n, self.groups, -1))
        g = T.cast(g, torch.float32) if g.dtype != torch.float32 else g
        mean = T.mean(g, dim=2, keepdim=True)
        d = g - mean
        y = d / T.sqrt(T.mean(d * d, dim=2, keepdim=True) + self.eps)
        per = (1, c) + (1,) * (len(shape) - 2)
        y = T.reshape(y, shape) * T.reshape(self.weight.value(), per) + T.reshape(self.bias.value(), per)
        return T.cast(y, x.dtype) if y.dtype != x.dtype else y


class _BatchNorm(Module):
    """Batch statistics while training, running statistics otherwise; the running
    update rides along with the forward pass as a side effect (``WithEffects``,
    tensor/autograd.go:759)."""

    def __init__(self, channels: int, eps: float = 1e-5, momentum: float = 0.1, dtype=torch.float32):
        self.weight = Param(torch.ones(channels, dtype=dtype), "weight")
        self.bias = Param(torch.zeros(channels, dtype=dtype), "bias")
        self.running_mean = Buffer(torch.zeros(channels), "running_mean")
        self.running_var = Buffer(torch.ones(channels), "running_var")
        self.eps, self.momentum = eps, momentum

    def forward(self, x):
        """Training: batch statistics normalise, and the new running statistics (momentum average of
        the old ones and the batch's mean / unbiased variance) are set on the buffers as recipes
        that the output carries as effects, so a backward pass computes them in its own schedule
        (nn/layers.go:196-243).  Evaluation: the running statistics normalise."""
        shape = tuple(x.shape)
        if len(shape) < 2:
            return T.core._error_tensor(T.ErrShape(f"batch norm of {shape}, want rank 2 or more"))
        c = shape[1]
        axes = tuple(d for d in range(len(shape)) if d != 1)
        bc = tuple(c if d == 1 else 1 for d in range(len(shape)))
        per = lambda t: T.reshape(t, bc)
        effects = ()
        if self.training:
            n = math.prod(shape) // max(c, 1)
            if n < 2:
                return T.core._error_tensor(T.ErrShape(
                    f"batch norm in training needs more than one value per channel, got {shape}"))
            xf = T.cast(x, torch.float32) if x.dtype != torch.float32 else x
            m = self.momentum
            if x._sharding is None:
                # one fused normalisation (and one fused backward) instead of eight elementwise passes;
                # the batch statistics for the running averages come from one more pass without autograd
                eps, dt = self.eps, x.dtype

                def bn(v, w, b):
                    return torch.nn.functional.batch_norm(v, None, None, w.to(v.dtype), b.to(v.dtype), True, 0.0, eps).to(dt)

                def stats(v):
                    var, mean = torch.var_mean(v.detach(), dim=axes, unbiased=False)
                    return torch.stack([mean, var])
                y = T.core._node(bn, (xf, self.weight.value(), self.bias.value()), {}, "batch_norm", known=(shape, x.dtype))
                mv = T.detach(T.core._node(stats, (xf,), {}, "batch_stats", known=((2, c), torch.float32)))
                new_mean = self.running_mean.value() * (1 - m) + mv[0] * m
                new_var = self.running_var.value() * (1 - m) + mv[1] * (m * n / (n - 1))
                self.running_mean.set(new_mean)
                self.running_var.set(new_var)
                return T.with_effects(y, new_mean, new_var)
            # on a device mesh the statistics are built from reductions the partitioner can split
            mean = T.mean(xf, dim=axes)
            d = xf - per(mean)
            var = T.mean(d * d, dim=axes)
            y = d / per(T.sqrt(var + self.eps))
            new_mean = self.running_mean.value() * (1 - m) + T.detach(mean) * m
            new_var = self.running_var.value() * (1 - m) + T.detach(var) * (m * n / (n - 1))
            self.running_mean.set(new_mean)
            self.running_var.set(new_var)
            effects = (new_mean, new_var)
        else:
            xf = T.cast(x, torch.float32) if x.dtype != torch.float32 else x
            y = (xf - per(self.running_mean.value())) / per(T.sqrt(self.running_var.value() + self.eps))
        y = y * per(self.weight.value()) + per(self.bias.value())
        if y.dtype != x.dtype:
            y = T.cast(y, x.dtype)
        return T.with_effects(y, *effects)


class BatchNorm1d(_BatchNorm):
    pass


class BatchNorm2d(_BatchNorm):
    pass


class Dropout(Module):
    """Mask drawn from the Philox stream of ``splitmix(seed ^ calls)`` (nn/layers.go:269-281)."""

    def __init__(self, p: float = 0.5, seed: int | None = None):
        self.p = p
        self._nn_skip_seed = _next_seed() if seed is None else seed
        self._nn_skip_calls = 0

    def forward(self, x):
        if not self.training or self.p == 0.0:
            return x
        self._nn_skip_calls += 1
        s = splitmix64(self._nn_skip_seed ^ self._nn_skip_calls)
        keep = 1.0 - self.p

        def run(v):
            if v.device.type == "meta":
                return torch.empty_like(v)
            mask = philox_uniform(tuple(v.shape), s, v.device) < keep
            return v * mask.to(v.dtype) / keep
        run._mimir_volatile = True   # the seed changes every call: kept out of the schedule's key
        return T.core._node(run, (x,), {}, "dropout", attrs={"kind": "unary"})


class _Fn(Module):
    def __init__(self, fn):
        self._nn_skip_fn = fn

    def forward(self, x):
        return self._nn_skip_fn(x)


def ReLU(): return _Fn(T.relu)
def GELU(): return _Fn(T.gelu)
def SiLU(): return _Fn(T.silu)
def Tanh(): return _Fn(T.tanh)
def Sigmoid(): return _Fn(T.sigmoid)
def Softmax(dim=-1): return _Fn(lambda x: T.softmax(x, dim))
def LeakyReLU(slope=0.01): return _Fn(lambda x: T.leaky_relu(x, slope))
def Flatten(): return _Fn(lambda x: T.reshape(x, (x.shape[0], -1)))
def MaxPool2d(kernel, stride=None, padding=0): return _Fn(lambda x: T.max_pool2d(x, kernel, stride, padding))
def AvgPool2d(kernel, stride=None, padding=0): return _Fn(lambda x: T.avg_pool2d(x, kernel, stride, padding))
def GlobalAvgPool(): return _Fn(lambda x: T.mean(x, dim=(2, 3)))
def Upsample(scale=2): return _Fn(lambda x: T.upsample_nearest(x, scale))
def Cast(dtype): return _Fn(lambda x: T.cast(x, dtype))


class Checkpoint(Module):
    """Wraps a module so that its activations are recomputed in backward (nn/checkpoint.go)."""

    def __init__(self, inner: Module):
        self.inner = inner

    def forward(self, x):
        # parameters enter the checkpointed function through the closure, so their
        # gradients still flow; only the activations are dropped and recomputed
        return self.inner(x) if not self.training else _checkpointed(self.inner, x)


def _checkpointed(inner, x):
    params = [p.value() for p in inner.parameters()]

    def run(v, *pv):
        if v.device.type == "meta":
            return T.core._meta_of(inner(T.core.Tensor(val=None, fn=None, shape=v.shape, dtype=v.dtype, device=x.device)))
        import torch.utils.checkpoint as cp

        def body(vv, *ps):
            memo = {id(t): p for t, p in zip(params, ps)}
            leaf = T.from_torch(vv)
            out = inner(leaf)
            # parameter leaves created inside ``inner`` are fresh objects: map them by storage
            for t, pp in T.autograd._collect_params(out).values():
                for q, val in zip(inner.parameters(), ps):
                    if pp is q:
                        memo[id(t)] = val
            (o,) = T.core.evaluate([out], memo, reuse_cached=True)
            return o
        if torch.is_grad_enabled():
            return cp.checkpoint(body, v, *pv, use_reentrant=False)
        return body(v, *pv)
    return T.core._node(run, (x, *params), {}, "checkpoint")


class LoRALinear(Module):
    """``base(x) + (alpha / r) * B A x`` with the base frozen (nn/lora.go)."""

    def __init__(self, base: Linear, rank: int = 8, alpha: float = 16.0):
        self.base = base
        for p in base.parameters():
            p.freeze()
        out_f, in_f = base.weight.shape
        self.lora_a = Param(normal_init((rank, in_f), 1.0 / rank, base.weight.dtype), "lora_a")
        self.lora_b = Param(torch.zeros(out_f, rank, dtype=base.weight.dtype), "lora_b")
        self.scale = alpha / rank

    def forward(self, x):
        return self.base(x) + T.matmul_t(T.matmul_t(x, self.lora_a.value()), self.lora_b.value()) * self.scale

    def merged_weight(self) -> torch.Tensor:
        return self.base.weight._data + self.scale * (self.lora_b._data @ self.lora_a._data)
