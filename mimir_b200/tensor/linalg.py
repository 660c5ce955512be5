"""Fourier transforms, linear algebra and the remaining elementwise / random ops of the tensor API
(reference: tensor/fft.go:39-137, tensor/linalg.go:53-340, tensor/elementwise.go, tensor/random.go).

Complex numbers are a trailing axis of 2 (real, imaginary), as the reference has them; transforms
work for any length along any axis.  The linear algebra (Cholesky, triangular and general solves,
inverse, determinant, QR, SVD, symmetric eigendecomposition) is batched over leading axes and
differentiable; like the reference's, it runs through a library (LAPACK on the host, cuSOLVER on
the GPU), not through kernels of this package.
"""
from __future__ import annotations

import torch

from . import core as C
from . import errors as E

_node = C._node


# ------------------------------------------------------------------ elementwise
exp2 = C._unary("exp2", torch.exp2)
log2 = C._unary("log2", torch.log2)
def greater(a, b):
    """``a > b`` elementwise (tensor.Greater): ``less`` with the operands swapped, so it traces and exports as one."""
    return C.less(b, a)
fmod = C._binary("fmod", torch.fmod)


# ------------------------------------------------------------------ Fourier
def _axis(t, axis, complex_in):
    nd = len(t.shape) - (1 if complex_in else 0)
    a = axis + nd if axis < 0 else axis
    if not 0 <= a < nd:
        raise IndexError
    return a


def _complex_op(name, fn, x, axis, complex_in=True, complex_out=True, **kw):
    if x._err is not None:
        return x
    if complex_in and (not x.shape or x.shape[-1] != 2):
        return C._error_tensor(E.ErrShape(f"{name}: complex input needs a trailing axis of 2, got {tuple(x.shape)}"))
    try:
        a = _axis(x, axis, complex_in)
    except IndexError:
        return C._error_tensor(E.ErrShape(f"{name}: axis {axis} out of range for {tuple(x.shape)}"))

    def run(v):
        z = torch.view_as_complex(v.float().contiguous()) if complex_in else v.float()
        out = fn(z, dim=a, **kw)
        return torch.view_as_real(out).to(v.dtype) if complex_out else out.to(v.dtype)
    return _node(run, (x,), {}, name, attrs={"axis": a})


def fft(x, axis: int = -1):
    """Discrete Fourier transform along ``axis`` of a tensor whose last axis holds (real, imaginary);
    ``axis`` counts the axes before that pair (tensor.FFT)."""
    return _complex_op("fft", torch.fft.fft, x, axis)


def ifft(x, axis: int = -1):
    return _complex_op("ifft", torch.fft.ifft, x, axis)


def rfft(x, axis: int = -1):
    """Transform of a real tensor: ``n // 2 + 1`` complex values along ``axis`` (a new trailing axis of 2)."""
    return _complex_op("rfft", torch.fft.rfft, x, axis, complex_in=False)


def irfft(x, axis: int = -1, n: int | None = None):
    """Inverse of ``rfft``: a real tensor of ``n`` values along ``axis`` (default ``2 (m - 1)``)."""
    return _complex_op("irfft", torch.fft.irfft, x, axis, complex_out=False, n=n)


# ------------------------------------------------------------------ linear algebra
def _square(name, x):
    if x._err is not None:
        return x
    if len(x.shape) < 2 or x.shape[-1] != x.shape[-2]:
        return C._error_tensor(E.ErrShape(f"{name}: needs square matrices, got {tuple(x.shape)}"))
    return None


def _lin(name, fn, *xs, outs: int = 1):
    def run(*vs):
        try:
            return fn(*[v.float() if v.dtype in (torch.bfloat16, torch.float16) else v for v in vs])
        except torch.linalg.LinAlgError as exc:
            raise E.ErrSingular(f"{name}: {exc}") from None
    return _node(run, xs, {}, name)


def cholesky(x):
    """Lower Cholesky factor of symmetric positive-definite matrices (``ErrSingular`` otherwise)."""
    return _square("cholesky", x) or _lin("cholesky", torch.linalg.cholesky, x)


def triangular_solve(a, b, upper: bool = False):
    """Solves ``a x = b`` for triangular ``a`` (the other triangle is ignored); ``b`` is a matrix
    ``[..., n, k]`` (tensor.TriangularSolve)."""
    bad = _square("triangular_solve", a)
    if bad is not None:
        return bad
    return _lin("triangular_solve", lambda p, q: torch.linalg.solve_triangular(torch.triu(p) if upper else torch.tril(p), q, upper=upper), a, b)


def solve(a, b):
    """Solves ``a x = b``; ``b`` is a matrix ``[..., n, k]`` or, for a single system, a vector ``[n]``."""
    return _square("solve", a) or _lin("solve", torch.linalg.solve, a, b)


def inv(x):
    return _square("inv", x) or _lin("inv", torch.linalg.inv, x)


def det(x):
    return _square("det", x) or _lin("det", torch.linalg.det, x)


def slogdet(x):
    """``(sign, log |det|)``."""
    bad = _square("slogdet", x)
    if bad is not None:
        return bad, bad
    return _lin("slogdet", lambda v: tuple(torch.linalg.slogdet(v)), x)


def qr(x):
    """Reduced QR: ``q [..., m, k]``, ``r [..., k, n]`` with ``k = min(m, n)``."""
    if x._err is not None:
        return x, x
    return _lin("qr", lambda v: tuple(torch.linalg.qr(v, mode="reduced")), x)


def svd(x):
    """Reduced SVD: ``u [..., m, k]``, ``s [..., k]``, ``vh [..., k, n]``."""
    if x._err is not None:
        return x, x, x
    return _lin("svd", lambda v: tuple(torch.linalg.svd(v, full_matrices=False)), x)


def eigh(x):
    """Eigenvalues (ascending) and eigenvectors of symmetric matrices (the lower triangle is read)."""
    bad = _square("eigh", x)
    if bad is not None:
        return bad, bad
    return _lin("eigh", lambda v: tuple(torch.linalg.eigh(v)), x)


# ------------------------------------------------------------------ random draws with a rate / shape parameter
def rand_gamma(alpha, seed: int = 0):
    """One Gamma(alpha, 1) draw per element of ``alpha``, reproducible from ``seed`` and
    differentiable in ``alpha`` (tensor.RandGamma)."""
    def run(a):
        if a.device.type == "meta":
            return torch.empty_like(a)
        g = torch.Generator(device=a.device).manual_seed(int(seed) & ((1 << 62) - 1))
        state = torch.get_rng_state() if a.device.type == "cpu" else torch.cuda.get_rng_state(a.device)
        try:
            (torch.set_rng_state if a.device.type == "cpu" else (lambda s: torch.cuda.set_rng_state(s, a.device)))(g.get_state())
            return torch._standard_gamma(a.float()).to(a.dtype)
        finally:
            (torch.set_rng_state if a.device.type == "cpu" else (lambda s: torch.cuda.set_rng_state(s, a.device)))(state)
    return C._volatile(_node(run, (alpha,), {}, "rand_gamma"))


def rand_poisson(rate, seed: int = 0):
    """One Poisson(rate) draw per element of ``rate`` (float counts), reproducible from ``seed``."""
    def run(r):
        if r.device.type == "meta":
            return torch.empty_like(r)
        g = torch.Generator(device=r.device).manual_seed(int(seed) & ((1 << 62) - 1))
        return torch.poisson(r.float(), generator=g).to(r.dtype)
    return C._volatile(_node(run, (rate,), {}, "rand_poisson"))


def from_slice(values, *shape, dtype=None, device=None):
    """A tensor of ``shape`` from a flat list of numbers (tensor.FromSlice); floats are float32, whole numbers int32."""
    v = torch.as_tensor(values)
    if dtype is None:
        dtype = torch.float32 if v.dtype.is_floating_point else (torch.bool if v.dtype == torch.bool else torch.int32)
    v = v.to(dtype)
    if shape and int(torch.tensor(shape).prod()) != v.numel():
        return C._error_tensor(E.ErrShape(f"from_slice: {v.numel()} values for shape {tuple(shape)}"))
    return C.tensor(v.reshape(tuple(shape)) if shape else v, dtype=dtype, device=device)


def scalar(value, dtype=None, device=None):
    """A tensor of no dimensions (tensor.Scalar)."""
    return from_slice(value, dtype=dtype, device=device)


def flatten(x, start: int = 1):
    """Every axis from ``start`` on as one (tensor.Flatten): ``[N, C, H, W] -> [N, C*H*W]`` by default."""
    s = tuple(x.shape)
    start = start if start >= 0 else len(s) + start
    return C.reshape(x, s[:start] + (-1,))
