"""Minimal PNG encoder (8-bit RGB or grey), so image workflows need no imaging library."""
from __future__ import annotations

import struct
import zlib

import numpy as np


def encode_png(chw) -> bytes:
    """``chw``: array [C, H, W] with C in (1, 3), values in [0, 1] or [-1, 1] (detected from the minimum)."""
    x = np.asarray(chw, dtype=np.float32)
    if x.ndim != 3 or x.shape[0] not in (1, 3):
        raise ValueError(f"encode_png wants [1 or 3, H, W], got {list(x.shape)}")
    lo = -1.0 if x.min() < 0 else 0.0
    x = np.clip((x - lo) / (1.0 - lo), 0.0, 1.0)
    img = (x * 255.0 + 0.5).astype(np.uint8).transpose(1, 2, 0)
    h, w, c = img.shape
    raw = b"".join(b"\x00" + img[r].tobytes() for r in range(h))

    def chunk(tag, data):
        return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)

    return (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2 if c == 3 else 0, 0, 0, 0)) +
            chunk(b"IDAT", zlib.compress(raw, 6)) + chunk(b"IEND", b""))
