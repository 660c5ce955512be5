"""Fused elementwise programs on the host (``csrc/cpu_fused.cc``): what the planner of
``tensor/plan.py`` emits for a chain of elementwise float32 ops on CPU tensors (reference:
internal/sched/fuse.go:200-362).  A program is ``[(op, dst, a, b), ...]`` over registers: inputs
first, then one register per instruction; an operand ``("c", value)`` is a constant."""
from __future__ import annotations

import ctypes

import torch

from .. import _native

CONST_BASE = 1 << 20
OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3, "maximum": 4, "minimum": 5,
       "neg": 16, "abs": 17, "relu": 18, "sqrt": 19, "rsqrt": 20, "recip": 21, "exp": 22, "log": 23, "tanh": 24, "sigmoid": 25,
       "silu": 26, "gelu": 27, "sin": 28, "cos": 29, "erf": 30, "log1p": 31, "expm1": 32, "sign": 33, "floor": 34, "ceil": 35,
       "softplus": 36}
BINARY = {"add", "sub", "mul", "div", "maximum", "minimum"}
_F = torch.nn.functional
TORCH = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div, "maximum": torch.maximum, "minimum": torch.minimum,
         "neg": torch.neg, "abs": torch.abs, "relu": torch.relu, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt, "recip": torch.reciprocal,
         "exp": torch.exp, "log": torch.log, "tanh": torch.tanh, "sigmoid": torch.sigmoid, "silu": _F.silu,
         "gelu": lambda v: _F.gelu(v, approximate="tanh"), "sin": torch.sin, "cos": torch.cos, "erf": torch.erf, "log1p": torch.log1p,
         "expm1": torch.expm1, "sign": torch.sign, "floor": torch.floor, "ceil": torch.ceil, "softplus": _F.softplus}


def _lib():
    lib = _native.lib()
    if not getattr(lib, "_fused_bound", False):
        c = ctypes
        lib.mimir_cpu_fused.argtypes = [c.c_void_p, c.c_int, c.c_void_p, c.c_void_p, c.c_int, c.c_void_p, c.c_int, c.c_void_p,
                                        c.c_void_p, c.c_int, c.c_longlong]
        lib._fused_bound = True
    return lib


class Fused:
    """A compiled elementwise program: ``names`` per instruction, operand pairs as register numbers
    (inputs ``0 .. n_in - 1``, then one register per instruction) and the result shape."""

    def __init__(self, instrs, n_in: int, shape):
        self.instrs, self.n_in, self.shape = list(instrs), n_in, tuple(shape)
        self.numel = 1
        for d in self.shape:
            self.numel *= int(d)
        code = []
        for k, (name, a, b) in enumerate(self.instrs):
            code += [OPS[name], n_in + k, a, b if b is not None else 0]
        self._code = (ctypes.c_int32 * len(code))(*code)
        self._out_reg = (ctypes.c_int * 1)(n_in + len(self.instrs) - 1)

    # -- execution
    def native_ok(self, vals) -> bool:
        if torch.is_grad_enabled() and any(v.requires_grad for v in vals):
            return False
        from ..tensor.memory import in_transform
        if in_transform():            # vmap / jvp wrapper tensors have no memory to hand to a kernel
            return False
        for v in vals:
            if v.device.type != "cpu" or v.dtype != torch.float32 or not v.is_contiguous() or v.numel() not in (self.numel, 1):
                return False
        return True

    def run_native(self, vals, out=None) -> torch.Tensor:
        if out is None:
            out = torch.empty(self.shape, dtype=torch.float32)
        n = len(vals)
        ptrs = (ctypes.c_void_p * max(n, 1))(*[v.data_ptr() for v in vals])
        scal = (ctypes.c_int * max(n, 1))(*[1 if (v.numel() == 1 and self.numel != 1) else 0 for v in vals])
        outs = (ctypes.c_void_p * 1)(out.data_ptr())
        rc = _lib().mimir_cpu_fused(self._code, len(self.instrs), ptrs, scal, n, None, 0, outs, self._out_reg, 1, self.numel)
        if rc:
            raise RuntimeError("fused elementwise program refused")
        return out

    def run_composed(self, vals) -> torch.Tensor:
        """The same program op by op in PyTorch (under autograd, or for operands the kernel does not take)."""
        regs = list(vals)
        for name, a, b in self.instrs:
            regs.append(TORCH[name](regs[a], regs[b]) if b is not None else TORCH[name](regs[a]))
        return regs[-1]

    def __call__(self, *vals):
        return self.run_native(vals) if self.native_ok(vals) else self.run_composed(vals)

    def into(self, *vals, out):
        if self.native_ok(vals) and out.is_contiguous() and out.dtype == torch.float32 and tuple(out.shape) == self.shape:
            self.run_native(vals, out)
        else:
            out.copy_(self.run_composed(vals))
