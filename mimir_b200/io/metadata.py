"""Typed metadata section of a ``.mim`` file ("MIMM").

Header: magic, u32 entry count, u64 pool bytes; 32-byte entries (u32 key offset,
u32 key length, u8 type, 3 pad, u32 count or byte count, u64 inline value or pool
offset, 8 reserved); then the pool.  Keys are sorted bytewise; every key is
followed in the pool by its out-of-line value.  Type codes: 1 uint64, 2 int64,
3 float64, 4 bool (all inline), 5 string, 7 int64 array, 8 float64 array,
9 string array (a table of (u32 offset, u32 length) pairs, then the bytes);
numeric arrays start on an 8-byte boundary.  Version 0.1 files use the magic "MMFM".  Python values map as: ``int`` -> int64
(``UInt64`` wrapper -> uint64), ``float``, ``bool``, ``str``, lists of those.
The reference reads the same keys through mimfile.Metadata (llm/model.go:77-94).
"""
from __future__ import annotations

import struct


class UInt64(int):
    """Marks an integer that is stored with the unsigned type code."""


def decode(section: bytes) -> dict:
    """Typed metadata section -> dict; a damaged section is a ``ValueError``."""
    try:
        return _decode(section)
    except (struct.error, IndexError, UnicodeDecodeError, OverflowError, MemoryError) as exc:
        raise ValueError(f"metadata section is damaged: {exc}") from None


def _decode(section: bytes) -> dict:
    if len(section) < 16 or section[:4] not in (b"MIMM", b"MMFM"):
        raise ValueError("not a metadata section")
    count, pool_bytes = struct.unpack_from("<IQ", section, 4)
    pool = section[16 + 32 * count: 16 + 32 * count + pool_bytes]
    out = {}
    for i in range(count):
        ko, kl, ty, c, val = struct.unpack_from("<IIB3xIQ", section, 16 + 32 * i)
        key = pool[ko:ko + kl].decode("utf-8")
        if ty == 1:
            out[key] = UInt64(val)
        elif ty == 2:
            out[key] = struct.unpack("<q", struct.pack("<Q", val))[0]
        elif ty == 3:
            out[key] = struct.unpack("<d", struct.pack("<Q", val))[0]
        elif ty == 4:
            out[key] = bool(val)
        elif ty == 5:
            out[key] = pool[val:val + c].decode("utf-8")
        elif ty == 7:
            out[key] = list(struct.unpack_from(f"<{c}q", pool, val))
        elif ty == 8:
            out[key] = list(struct.unpack_from(f"<{c}d", pool, val))
        elif ty == 9:
            tab = [struct.unpack_from("<II", pool, val + 8 * j) for j in range(c)]
            out[key] = [pool[o:o + l].decode("utf-8", errors="surrogateescape") for o, l in tab]
        else:
            raise ValueError(f"metadata key {key!r}: unknown type code {ty}")
    return out


def encode(md: dict, magic: bytes = b"MIMM") -> bytes:
    items = sorted(((k.encode("utf-8"), v) for k, v in md.items()), key=lambda kv: kv[0])
    pool = bytearray()
    entries = []

    def align8():
        while len(pool) % 8:
            pool.append(0)

    for key, v in items:
        ko = len(pool)
        pool += key
        if isinstance(v, bool):
            entries.append((ko, len(key), 4, 0, int(v)))
        elif isinstance(v, UInt64):
            entries.append((ko, len(key), 1, 0, int(v)))
        elif isinstance(v, int):
            entries.append((ko, len(key), 2, 0, struct.unpack("<Q", struct.pack("<q", v))[0]))
        elif isinstance(v, float):
            entries.append((ko, len(key), 3, 0, struct.unpack("<Q", struct.pack("<d", v))[0]))
        elif isinstance(v, str):
            b = v.encode("utf-8")
            entries.append((ko, len(key), 5, len(b), len(pool)))
            pool += b
        elif isinstance(v, (list, tuple)):
            if v and all(isinstance(x, str) for x in v):
                bs = [x.encode("utf-8", errors="surrogateescape") for x in v]
                start = len(pool)  # string tables are not aligned
                off = start + 8 * len(bs)
                for b in bs:
                    pool += struct.pack("<II", off, len(b))
                    off += len(b)
                for b in bs:
                    pool += b
                entries.append((ko, len(key), 9, len(bs), start))
            elif all(isinstance(x, int) and not isinstance(x, bool) for x in v):
                align8()
                entries.append((ko, len(key), 7, len(v), len(pool)))
                pool += struct.pack(f"<{len(v)}q", *v)
            else:
                align8()
                entries.append((ko, len(key), 8, len(v), len(pool)))
                pool += struct.pack(f"<{len(v)}d", *[float(x) for x in v])
        else:
            raise TypeError(f"metadata value of {key!r} has unsupported type {type(v).__name__}")
    out = bytearray(magic + struct.pack("<IQ", len(entries), len(pool)))
    for ko, kl, ty, c, val in entries:
        out += struct.pack("<IIB3xIQQ", ko, kl, ty, c, val, 0)
    return bytes(out + pool)
