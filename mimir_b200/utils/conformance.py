"""One table of cases for every backend, and the oracle files made from it.

Two jobs of the reference meet here.  Its kernel conformance harness runs the same ``Case`` list on
every backend and compares with the CPU backend (backend/internal/kerneltest/kerneltest.go:58-120);
its golden generator draws seeded inputs, computes the expected results with a float64 oracle and
stores ``<case>/in<i>``, ``<case>/out``, ``<case>/gout`` and ``<case>/grad<i>`` as tensors of ``.mim``
files (tools/golden/gen.py:1-60).  Here one table serves both:

* ``generate(out_dir)`` writes the oracle files (PyTorch float64 on the CPU, rounded to float32;
  inputs from this package's Philox stream, which is the same on every device);
* ``check(dir, device, dtype)`` runs every case through the public lazy tensor API on a device and
  compares with the stored results: float32 on the CPU and on the GPU (PyTorch's CUDA kernels), and
  bfloat16 on the GPU, where matmul / linear / attention / norms / activations / conv / pooling /
  embedding run this package's native sm_100a kernels;
* ``python -m mimir_b200.utils.conformance --out DIR [--check] [--device gpu] [--dtype bf16]``.

A case: ``name``, ``run`` over lazy tensors, ``oracle`` over float64 torch tensors, input specs
(shape and kind), whether gradients are part of it, and tolerances for float32 and bfloat16 (a
fraction of the largest expected magnitude, plus a per-row bound so that an error confined to one
row or tile edge does not hide behind a large value elsewhere).
"""
from __future__ import annotations

import argparse
import math
import os
from dataclasses import dataclass, field

import torch

from .. import tensor as T
from ..io import mim
from ..tensor.random import philox_normal, philox_uniform

F = torch.nn.functional


@dataclass
class Case:
    name: str
    run: object                      # lazy tensors -> lazy tensor
    oracle: object                   # float64 / int64 torch tensors -> torch tensor
    inputs: list                     # (shape, kind): "n" normal, "p" positive, "u" in (0, 1), "i<C>" ints below C, "b" bool
    grad: bool = True
    tol32: float = 2e-5
    tol16: float = 2.5e-2
    file: str = "ops"
    half: bool = True                # part of the bfloat16 pass
    notes: str = ""
    skip_grad_inputs: tuple = field(default_factory=tuple)


def _draw(shape, kind, seed):
    if kind == "n":
        return philox_normal(shape, seed, "cpu")
    if kind == "p":
        return philox_uniform(shape, seed, "cpu") * 2.0 + 0.25
    if kind == "u":
        return philox_uniform(shape, seed, "cpu") * 0.98 + 0.01
    if kind == "b":
        return philox_uniform(shape, seed, "cpu") > 0.5
    if kind.startswith("i"):
        return (philox_uniform(shape, seed, "cpu") * int(kind[1:])).long().clamp_(0, int(kind[1:]) - 1)
    raise ValueError(kind)


def _sdpa(q, k, v, causal):
    if k.shape[1] != q.shape[1]:
        k = k.repeat_interleave(q.shape[1] // k.shape[1], 1)
        v = v.repeat_interleave(q.shape[1] // v.shape[1], 1)
    s = q @ k.transpose(-1, -2) / math.sqrt(q.shape[-1])
    if causal:
        Tq, Tk = s.shape[-2:]
        i, j = torch.arange(Tq)[:, None], torch.arange(Tk)[None]
        s = s.masked_fill(j > i + (Tk - Tq), float("-inf"))
    return torch.softmax(s, -1) @ v


def _rms(x, g, eps=1e-5):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * g


def _cases() -> list:
    C = Case
    E = [("n", T.neg, torch.neg), ("exp", T.exp, torch.exp), ("sin", T.sin, torch.sin), ("cos", T.cos, torch.cos),
         ("tanh", T.tanh, torch.tanh), ("sigmoid", T.sigmoid, torch.sigmoid), ("relu", T.relu, torch.relu),
         ("silu", T.silu, F.silu), ("abs", T.abs_, torch.abs), ("erf", T.erf, torch.erf),
         ("gelu", T.gelu, lambda x: F.gelu(x, approximate="tanh")), ("softplus", T.softplus, F.softplus)]
    out = [C("unary_" + n, f, o, [((6, 40), "n")]) for n, f, o in E]
    P = [("log", T.log, torch.log), ("sqrt", T.sqrt, torch.sqrt), ("rsqrt", T.rsqrt, torch.rsqrt), ("recip", T.recip, torch.reciprocal),
         ("log1p", T.log1p, torch.log1p), ("lgamma", T.lgamma, torch.lgamma)]
    out += [C("unary_" + n, f, o, [((6, 40), "p")]) for n, f, o in P]
    B = [("add", T.add, torch.add), ("sub", T.sub, torch.sub), ("mul", T.mul, torch.mul), ("maximum", T.maximum, torch.maximum),
         ("minimum", T.minimum, torch.minimum)]
    out += [C("binary_" + n, f, o, [((4, 1, 24), "n"), ((5, 24), "n")]) for n, f, o in B]
    out += [
        C("binary_div", T.div, torch.div, [((4, 24), "n"), ((4, 24), "p")]),
        C("binary_pow", T.pow_, torch.pow, [((4, 24), "p"), ((4, 24), "n")], tol16=6e-2),
        C("where", lambda c, a, b: T.where(c, a, b), lambda c, a, b: torch.where(c, a, b), [((5, 16), "b"), ((5, 16), "n"), ((5, 16), "n")]),
        C("clamp", lambda x: T.clamp(x, -0.5, 0.7), lambda x: x.clamp(-0.5, 0.7), [((8, 16), "n")], half=False,
          notes="rounding an input across a bound flips its gradient"),
        C("sum_all", lambda x: T.sum_(x), lambda x: x.sum(), [((3, 8, 16), "n")], tol16=4e-2),
        C("sum_axis1", lambda x: T.sum_(x, 1), lambda x: x.sum(1), [((3, 8, 16), "n")]),
        C("mean_last_keep", lambda x: T.mean(x, -1, True), lambda x: x.mean(-1, keepdim=True), [((3, 8, 16), "n")]),
        C("max_axis2", lambda x: T.max_(x, 2), lambda x: x.amax(2), [((3, 8, 16), "n")]),
        C("min_axis0", lambda x: T.min_(x, 0), lambda x: x.amin(0), [((3, 8, 16), "n")]),
        C("var_axis1", lambda x: T.var(x, 1), lambda x: x.var(1, unbiased=True), [((3, 8, 16), "n")], tol16=5e-2),
        C("logsumexp_last", lambda x: T.logsumexp(x, -1), lambda x: torch.logsumexp(x, -1), [((6, 32), "n")]),
        C("softmax_axis1", lambda x: T.softmax(x, 1), lambda x: torch.softmax(x, 1), [((4, 16, 8), "n")]),
        C("log_softmax_large", lambda x: T.log_softmax(x * 30.0, -1), lambda x: torch.log_softmax(x * 30.0, -1), [((6, 48), "n")], tol16=4e-2),
        C("cumsum_axis1", lambda x: T.cumsum(x, 1), lambda x: x.cumsum(1), [((4, 24), "n")], tol16=5e-2),
        C("reshape_permute", lambda x: T.permute(T.reshape(x, (4, 6, 8)), (2, 0, 1)), lambda x: x.reshape(4, 6, 8).permute(2, 0, 1), [((24, 8), "n")]),
        C("expand_mul", lambda x, y: T.expand(x, (5, 4, 16)) * y, lambda x, y: x.expand(5, 4, 16) * y, [((1, 4, 16), "n"), ((5, 4, 16), "n")]),
        C("pad_shrink", lambda x: T.shrink(T.pad(x, ((1, 2), (0, 3))), ((1, 6), (2, 15))), lambda x: F.pad(x, (0, 3, 1, 2))[1:6, 2:15], [((5, 16), "n")]),
        C("cat_split", lambda a, b: T.split(T.cat([a, b], 1), [10, 14], 1)[1], lambda a, b: torch.cat([a, b], 1).split([10, 14], 1)[1], [((4, 8), "n"), ((4, 16), "n")]),
        C("flip_transpose", lambda x: T.transpose(T.flip(x, (1,)), 0, 1), lambda x: x.flip(1).transpose(0, 1), [((6, 16), "n")]),
        C("gather_axis1", lambda x, i: T.gather(x, 1, i), lambda x, i: x.gather(1, i), [((6, 16), "n"), ((6, 4), "i16")]),
        C("one_hot_matmul", lambda i, w: T.matmul(T.one_hot(i, 16, w.dtype), w), lambda i, w: F.one_hot(i, 16).double() @ w, [((12,), "i16"), ((16, 8), "n")]),
        C("gather_rows", lambda w, i: T.gather_rows(w, i), lambda w, i: w[i], [((32, 64), "n"), ((4, 24), "i32")]),
        C("matmul_2d", T.matmul, torch.matmul, [((64, 96), "n"), ((96, 40), "n")], tol32=5e-5),
        C("matmul_batched", T.matmul, torch.matmul, [((3, 32, 64), "n"), ((3, 64, 24), "n")], tol32=5e-5),
        C("linear_bias", lambda x, w, b: T.matmul_t(x, w, b), lambda x, w, b: x @ w.t() + b, [((4, 32, 64), "n"), ((128, 64), "n"), ((128,), "n")], tol32=5e-5, file="nn"),
        C("linear_gelu_residual", lambda x, w, b, r: T.gelu(T.matmul_t(x, w, b)) + r,
          lambda x, w, b, r: F.gelu(x @ w.t() + b, approximate="tanh") + r, [((64, 64), "n"), ((64, 64), "n"), ((64,), "n"), ((64, 64), "n")], tol32=5e-5, file="nn"),
        C("swiglu", lambda g, u: T.silu(g) * u, lambda g, u: F.silu(g) * u, [((16, 64), "n"), ((16, 64), "n")], file="nn"),
        C("layer_norm", lambda x, g, b: T.layer_norm(x, g, b, 1e-5), lambda x, g, b: F.layer_norm(x, (64,), g, b, 1e-5), [((4, 24, 64), "n"), ((64,), "p"), ((64,), "n")], file="nn", tol16=4e-2),
        C("rms_norm", lambda x, g: T.rms_norm(x, g, 1e-5), _rms, [((4, 24, 64), "n"), ((64,), "p")], file="nn", tol16=4e-2),
        C("attention_causal", lambda q, k, v: T.attention(q, k, v, causal=True), lambda q, k, v: _sdpa(q, k, v, True),
          [((2, 4, 128, 64), "n"), ((2, 4, 128, 64), "n"), ((2, 4, 128, 64), "n")], file="attention", tol32=2e-3, tol16=4e-2),
        C("attention_gqa_cross", lambda q, k, v: T.attention(q, k, v), lambda q, k, v: _sdpa(q, k, v, False),
          [((1, 4, 48, 64), "n"), ((1, 2, 80, 64), "n"), ((1, 2, 80, 64), "n")], file="attention", tol32=2e-3, tol16=4e-2),
        C("conv2d_3x3_pad1", lambda x, w, b: T.conv2d(x, w, b, padding=1), lambda x, w, b: F.conv2d(x, w, b, padding=1),
          [((2, 8, 12, 12), "n"), ((16, 8, 3, 3), "n"), ((16,), "n")], file="nn", tol32=1e-4, tol16=4e-2),
        C("max_pool_2x2", lambda x: T.max_pool2d(x, 2), lambda x: F.max_pool2d(x, 2), [((2, 8, 12, 12), "n")], file="nn"),
        C("avg_pool_2x2", lambda x: T.avg_pool2d(x, 2), lambda x: F.avg_pool2d(x, 2), [((2, 8, 12, 12), "n")], file="nn"),
    ]
    from ..nn import loss as L
    out += [
        C("loss_cross_entropy", L.cross_entropy, lambda l, t: F.cross_entropy(l, t), [((16, 32), "n"), ((16,), "i32")], file="nn", half=False),
        C("loss_mse", L.mse, F.mse_loss, [((8, 16), "n"), ((8, 16), "n")], file="nn", skip_grad_inputs=(1,)),
        C("loss_bce_with_logits", L.bce_with_logits, F.binary_cross_entropy_with_logits, [((8, 16), "n"), ((8, 16), "u")], file="nn", skip_grad_inputs=(1,)),
        C("loss_huber", L.huber, lambda p, t: F.huber_loss(p, t, delta=1.0), [((8, 16), "n"), ((8, 16), "n")], file="nn", skip_grad_inputs=(1,)),
    ]
    names = [c.name for c in out]
    assert len(names) == len(set(names))
    return out


CASES = _cases()
FILES = sorted({c.file for c in CASES})


def _inputs(case: Case, idx: int):
    return [_draw(shape, kind, 1000 * (idx + 1) + k) for k, (shape, kind) in enumerate(case.inputs)]


def generate(out_dir: str) -> dict:
    """Writes one ``.mim`` per file name of the table; returns {file: number of cases}."""
    os.makedirs(out_dir, exist_ok=True)
    per_file: dict = {f: {} for f in FILES}
    for idx, c in enumerate(CASES):
        ins = _inputs(c, idx)
        wide = [x.double().requires_grad_(c.grad and x.dtype.is_floating_point and k not in c.skip_grad_inputs) if x.dtype.is_floating_point else x
                for k, x in enumerate(ins)]
        out = c.oracle(*wide)
        tensors = per_file[c.file]
        for k, x in enumerate(ins):
            tensors[f"{c.name}/in{k}"] = x.to(torch.int32) if x.dtype == torch.int64 else (x.to(torch.uint8) if x.dtype == torch.bool else x)
        tensors[f"{c.name}/out"] = out.detach().float()
        if c.grad:
            gout = philox_normal(tuple(out.shape), 777 + idx, "cpu") if out.dim() else torch.ones(())
            tensors[f"{c.name}/gout"] = gout
            need = [w for w in wide if torch.is_tensor(w) and w.requires_grad]
            grads = torch.autograd.grad(out, need, gout.double(), allow_unused=True)
            it = iter(grads)
            for k, w in enumerate(wide):
                if torch.is_tensor(w) and w.requires_grad:
                    g = next(it)
                    tensors[f"{c.name}/grad{k}"] = (torch.zeros_like(w) if g is None else g).float()
    meta = {"oracle": "torch-float64", "torch": torch.__version__, "generator": "mimir_b200.utils.conformance"}
    for f, tensors in per_file.items():
        mim.write_tensors(os.path.join(out_dir, f + ".mim"), tensors, metadata=meta)
    return {f: sum(1 for c in CASES if c.file == f) for f in FILES}


def _close(got, want, tol, what):
    got, want = got.detach().double().cpu(), want.double()
    if tuple(got.shape) != tuple(want.shape):
        return f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    if not want.numel():
        return None
    scale = max(float(want.abs().max()), 1e-3)
    err = (got - want).abs()
    if not torch.isfinite(got).all() and torch.isfinite(want).all():
        return f"{what}: non-finite values"
    if float(err.max()) > tol * scale + tol * 1e-2:
        return f"{what}: max error {float(err.max()):.3g} against {tol * scale:.3g} (scale {scale:.3g})"
    if want.dim() >= 2:
        # the same bound against each row's own magnitude, with slack for rows of small values
        rows_w = want.reshape(-1, want.shape[-1]).abs().amax(1)
        rows_e = err.reshape(-1, want.shape[-1]).amax(1)
        bad = rows_e > tol * 4 * (rows_w + 0.1 * scale)
        if bool(bad.any()):
            r = int(bad.nonzero()[0])
            return f"{what}: row {r} error {float(rows_e[r]):.3g} against its magnitude {float(rows_w[r]):.3g}"
    return None


def check(golden_dir: str, device=None, dtype=torch.float32, only=None) -> list:
    """Runs the table on ``device`` in ``dtype`` against the stored oracle results; returns a list of
    failure messages (empty = conformant)."""
    from ..tensor.autograd import Param, backward
    device = device or T.CPU()
    half = dtype != torch.float32
    failures = []
    files = {f: mim.open(os.path.join(golden_dir, f + ".mim")) for f in FILES}
    try:
        for c in CASES:
            if (only and c.name not in only) or (half and not c.half):
                continue
            m = files[c.file]
            tol = c.tol16 if half else c.tol32
            ins = []
            k = 0
            while f"{c.name}/in{k}" in m:
                ins.append(m.tensor(f"{c.name}/in{k}").clone())
                k += 1
            params, args = [], []
            for k, (x, (_, kind)) in enumerate(zip(ins, c.inputs)):
                if kind == "b":
                    args.append(T.tensor(x.bool(), device=device))
                elif kind.startswith("i"):
                    args.append(T.tensor(x.long(), device=device))
                else:
                    p = Param(x.to(dtype).to(device.torch))
                    params.append((k, p))
                    args.append(p.value())
            try:
                out = c.run(*args)
                if out.err is not None:
                    failures.append(f"{c.name}: {type(out.err).__name__}: {out.err}")
                    continue
                with_grad = c.grad and f"{c.name}/gout" in m and params
                if with_grad:
                    # backward first: it walks the graph below ``out``, which realizing ``out`` would drop
                    gout = T.tensor(m.tensor(f"{c.name}/gout").clone().to(out.dtype), device=device)
                    backward(T.sum_(T.cast(out, T.float32) * T.cast(gout, T.float32)))
                msg = _close(out.data(), m.tensor(f"{c.name}/out"), tol, f"{c.name}/out")
                if msg:
                    failures.append(msg)
                    continue
                if with_grad:
                    for k, p in params:
                        name = f"{c.name}/grad{k}"
                        if name not in m:
                            continue
                        g = p.grad()
                        if g is None:
                            failures.append(f"{name}: no gradient")
                            continue
                        msg = _close(g.data(), m.tensor(name), tol * 2, name)
                        if msg:
                            failures.append(msg)
            except T.MimirError as e:
                failures.append(f"{c.name}: {type(e).__name__}: {e}")
    finally:
        for f in files.values():
            f.close()
    return failures


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", required=True, help="directory of the oracle files")
    ap.add_argument("--check", action="store_true", help="run the table against the files instead of writing them")
    ap.add_argument("--device", default="cpu", choices=["cpu", "gpu"])
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16"])
    a = ap.parse_args(argv)
    if not a.check:
        for f, n in generate(a.out).items():
            print(f"{f}.mim: {n} cases")
        return 0
    dev = T.GPU(0) if a.device == "gpu" else T.CPU()
    bad = check(a.out, dev, torch.bfloat16 if a.dtype == "bf16" else torch.float32)
    for line in bad:
        print("FAIL", line)
    print(f"{len(CASES)} cases, {len(bad)} failures on {a.device} in {a.dtype}")
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
