"""Fused attention forward / backward (``csrc/attention_sm100.cu``).

Reference surface: ``tensor.Attention`` with ``Causal``, ``CausalOffset`` and
grouped-query heads (tensor/attention.go:81-253); logsumexp is returned so the
backward pass can recompute probabilities (backend/op.go:117-135).
"""
from __future__ import annotations

import math

import torch

from .. import _native
from ._util import ptr, stream_ptr


def attention_fwd(q, k, v, out, lse, *, causal=True, offset=None, scale=None):
    """q [B,Tq,Hq,D], k/v [B,Tk,Hkv,D] (bf16, last dim contiguous, any token pitch)."""
    B, Tq, Hq, D = q.shape
    _, Tk, Hkv, _ = k.shape
    if offset is None:
        offset = Tk - Tq
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    rc = _native.lib().mimir_attention_fwd(
        ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse), B, Tq, Tk, Hq, Hkv, D, q.stride(1), k.stride(1),
        v.stride(1), out.stride(1), int(causal), int(offset), float(scale), stream_ptr())
    _native.check(rc, "attention_fwd")
    return out


def attention_bwd(q, k, v, out, dout, lse, dsum, dq, dk, dv, *, causal=True, offset=None, scale=None):
    B, Tq, Hq, D = q.shape
    _, Tk, Hkv, _ = k.shape
    if offset is None:
        offset = Tk - Tq
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if dk.stride(1) != dv.stride(1):
        raise ValueError("dk and dv must share a token pitch")
    rc = _native.lib().mimir_attention_bwd(
        ptr(q), ptr(k), ptr(v), ptr(out), ptr(dout), ptr(lse), ptr(dsum), ptr(dq), ptr(dk), ptr(dv),
        B, Tq, Tk, Hq, Hkv, D, q.stride(1), k.stride(1), v.stride(1), out.stride(1), dout.stride(1),
        dq.stride(1), dk.stride(1), int(causal), int(offset), float(scale), stream_ptr())
    _native.check(rc, "attention_bwd")


def _split_packed(qkv, B, T, Hq, Hkv, D):
    """Views of a fused projection output [B*T, (Hq + 2 Hkv) D] as q, k, v."""
    x = qkv.view(B, T, (Hq + 2 * Hkv) * D)
    q = x[:, :, : Hq * D].unflatten(2, (Hq, D))
    k = x[:, :, Hq * D: (Hq + Hkv) * D].unflatten(2, (Hkv, D))
    v = x[:, :, (Hq + Hkv) * D:].unflatten(2, (Hkv, D))
    return q, k, v


def attention_fwd_packed(qkv, out, lse, B, T, Hq, Hkv, D, causal=True):
    q, k, v = _split_packed(qkv, B, T, Hq, Hkv, D)
    return attention_fwd(q, k, v, out.view(B, T, Hq, D), lse, causal=causal)


def attention_bwd_packed(qkv, out, dout, lse, dsum, dqkv, B, T, Hq, Hkv, D, causal=True):
    q, k, v = _split_packed(qkv, B, T, Hq, Hkv, D)
    dq, dk, dv = _split_packed(dqkv, B, T, Hq, Hkv, D)
    attention_bwd(q, k, v, out.view(B, T, Hq, D), dout.view(B, T, Hq, D), lse, dsum, dq, dk, dv,
                  causal=causal)
