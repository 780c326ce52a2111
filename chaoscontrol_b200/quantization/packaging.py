"""int6 + LZMA container: ``lzma(torch.save({"w": quantized, "m": meta}))``."""
from __future__ import annotations

import io
import lzma

import torch

LZMA_PRESET = 9


def pack_int6_lzma(quantized: dict, meta: dict, *, preset: int = LZMA_PRESET) -> bytes:
    buf = io.BytesIO()
    torch.save({"w": quantized, "m": meta}, buf)
    return lzma.compress(buf.getvalue(), preset=preset)


def unpack_int6_lzma(blob: bytes, *, map_location="cpu"):
    try:
        payload = torch.load(io.BytesIO(lzma.decompress(blob)), map_location=map_location,
                             weights_only=False)
    except Exception as exc:
        raise ValueError(f"blob is not a valid int6-lzma container: {exc}") from exc
    if not isinstance(payload, dict) or "w" not in payload or "m" not in payload:
        raise ValueError("blob is not a valid int6-lzma container")
    return payload["w"], payload["m"]
