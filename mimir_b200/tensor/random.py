"""Counter-based random numbers: Philox4x32-10, identical on every device.

Element ``i`` of a stream is word ``i % 4`` of the Philox block with counter
``i // 4`` and key ``(seed_lo, seed_hi)`` (reference: backend/cpu/rand.go,
backend/internal/gen/gen.go:577-610).  Uniforms use the top 24 bits; normals use
Box-Muller on pairs of uniforms with ``cospi`` / ``sinpi``.  The generator runs
as vectorised integer tensor arithmetic on the target device, so CPU and GPU
produce bit-identical streams (dropout masks must match across devices).
"""
from __future__ import annotations

import math

import torch

_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def _mul32(a: torch.Tensor, m: int):
    """(hi, lo) 32-bit halves of a * m for 0 <= a < 2^32 held in int64."""
    a_lo, a_hi = a & 0xFFFF, a >> 16
    m_lo, m_hi = m & 0xFFFF, m >> 16
    ll = a_lo * m_lo
    lh = a_lo * m_hi
    hl = a_hi * m_lo
    hh = a_hi * m_hi
    mid = (ll >> 16) + (lh & 0xFFFF) + (hl & 0xFFFF)
    lo = ((mid & 0xFFFF) << 16) | (ll & 0xFFFF)
    hi = hh + (lh >> 16) + (hl >> 16) + (mid >> 16)
    return hi & _MASK, lo & _MASK


def philox_blocks(nblocks: int, seed: int, device, first_block: int = 0) -> torch.Tensor:
    """[nblocks, 4] int64 tensor of 32-bit words."""
    ctr = torch.arange(first_block, first_block + nblocks, dtype=torch.int64, device=device)
    c0, c1 = ctr & _MASK, (ctr >> 32) & _MASK
    c2 = torch.zeros_like(ctr)
    c3 = torch.zeros_like(ctr)
    k0, k1 = seed & _MASK, (seed >> 32) & _MASK
    for _ in range(10):
        hi0, lo0 = _mul32(c0, _M0)
        hi1, lo1 = _mul32(c2, _M1)
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & _MASK, lo1, (hi0 ^ c3 ^ k1) & _MASK, lo0
        k0, k1 = (k0 + _W0) & _MASK, (k1 + _W1) & _MASK
    return torch.stack([c0, c1, c2, c3], 1)


def philox_words(n: int, seed: int, device) -> torch.Tensor:
    return philox_blocks((n + 3) // 4, seed, device).reshape(-1)[:n]


def philox_uniform(shape, seed: int, device) -> torch.Tensor:
    n = math.prod(shape)
    w = philox_words(n, seed, device)
    return ((w >> 8).to(torch.float32) * (1.0 / (1 << 24))).reshape(shape)


def philox_normal(shape, seed: int, device) -> torch.Tensor:
    n = math.prod(shape)
    pairs = (n + 1) // 2
    w = philox_words(2 * pairs, seed, device).reshape(pairs, 2)
    u1 = ((w[:, 0] >> 8).to(torch.float32) + 1.0) * (1.0 / (1 << 24))  # (0, 1]
    u2 = (w[:, 1] >> 8).to(torch.float32) * (1.0 / (1 << 24))
    r = torch.sqrt(-2.0 * torch.log(u1))
    z = torch.stack([r * torch.cos(2 * math.pi * u2), r * torch.sin(2 * math.pi * u2)], 1).reshape(-1)[:n]
    return z.reshape(shape)


def splitmix64(x: int) -> int:
    """Seed derivation used by ``nn`` (nn/nn.go:252-268): dropout seed = splitmix(seed ^ calls)."""
    x = (x + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return z ^ (z >> 31)
