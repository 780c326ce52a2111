"""Self-describing controller weight files (CSWG version 3).

Byte layout, shared with the reference's writer (experiments/25_controller_pretrain/dump_to_cpp.py:17-175) so
files travel both ways: a 20-byte little-endian header ``magic "CSWG" | version 3 | dtype code 1 (fp16) |
manifest bytes | 0``, a compact JSON manifest (``dims`` of the policy and, per tensor, name / shape / dtype /
offset / nbytes relative to the payload), then the fp16 payload.  A reader needs no fixed tensor order: the
residual attention branch and the bucket embedding are present when the manifest lists them with data.

:func:`policy_to_cswg` / :func:`policy_from_cswg` map the native policy's flat fp32 vector
(``[W_vp | b_vp | W_lh | b_lh | W_sb | alpha]``, then ``[lambda | W_q | W_k | W_v | W_o | W_e]`` when it has
heads, then the bucket embedding) onto the fourteen named tensors and back.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Any

import numpy as np

MAGIC = b"CSWG"
VERSION = 3
DTYPE_FP16 = 1
_HEADER = struct.Struct("<4sIIII")
HEADER_SIZE = _HEADER.size
TENSOR_NAMES = ("W_vp", "b_vp", "W_lh", "b_lh", "W_sb", "alpha", "temperature", "bucket_embed", "lambda_hxh", "W_q", "W_k",
                "W_v", "W_o", "W_e")
DIM_KEYS = ("n_vertices", "k_v", "k_e", "k_s", "h", "n_heads", "n_buckets", "bucket_embed_dim")

__all__ = ["write_cswg_v3", "load_cswg_v3", "file_version", "policy_to_cswg", "policy_from_cswg", "tensor_shapes",
           "TENSOR_NAMES", "VERSION"]


def tensor_shapes(dims: dict[str, int]) -> dict[str, tuple[int, ...]]:
    kv, ke, ks, h, nh = (int(dims[k]) for k in ("k_v", "k_e", "k_s", "h", "n_heads"))
    nb, ed = int(dims["n_buckets"]), int(dims["bucket_embed_dim"])
    return {"W_vp": (kv, h), "b_vp": (h,), "W_lh": (h,), "b_lh": (), "W_sb": (ks,), "alpha": (), "temperature": (),
            "bucket_embed": (nb, ed), "lambda_hxh": (), "W_q": (nh, h, h), "W_k": (nh, h, h), "W_v": (nh, h, h),
            "W_o": (nh, h), "W_e": (nh, ke)}


def write_cswg_v3(path: Path | str, tensors: dict[str, Any], dims: dict[str, int]) -> dict[str, Any]:
    """Writes the fourteen tensors (fp32 in, fp16 on disk) and returns the manifest with file statistics."""
    missing = [n for n in TENSOR_NAMES if n not in tensors]
    if missing:
        raise KeyError(f"missing tensor(s) {missing}; have {sorted(tensors)}")
    entries, parts, off, drift = [], [], 0, 0.0
    for name in TENSOR_NAMES:
        t = np.asarray(tensors[name], dtype=np.float32)
        half = np.ascontiguousarray(t.astype(np.float16))
        if t.size:
            drift = max(drift, float(np.abs(t - half.astype(np.float32)).max()))
        raw = half.tobytes(order="C")
        entries.append({"name": name, "shape": list(t.shape), "dtype": "fp16", "offset": off, "nbytes": len(raw)})
        parts.append(raw)
        off += len(raw)
    manifest = {"magic": "CSWG", "version": VERSION, "dtype_code": DTYPE_FP16, "dtype": "fp16",
                "dims": {k: int(dims[k]) for k in DIM_KEYS}, "tensors": entries}
    blob = json.dumps(manifest, sort_keys=True, separators=(",", ":")).encode()
    out = Path(path)
    out.parent.mkdir(parents=True, exist_ok=True)
    with out.open("wb") as fh:
        fh.write(_HEADER.pack(MAGIC, VERSION, DTYPE_FP16, len(blob), 0))
        fh.write(blob)
        for p in parts:
            fh.write(p)
    return {**manifest, "path": str(out), "header_bytes": HEADER_SIZE, "manifest_bytes": len(blob), "payload_bytes": off,
            "file_bytes": HEADER_SIZE + len(blob) + off, "fp32_vs_fp16_max_abs_drift": drift}


def file_version(path: Path | str) -> int:
    """Version field of a CSWG file's header; raises on a foreign file."""
    with open(path, "rb") as fh:
        head = fh.read(8)
    if len(head) < 8 or head[:4] != MAGIC:
        raise ValueError(f"{path}: not a CSWG file")
    return int(struct.unpack("<I", head[4:8])[0])


def load_cswg_v3(path: Path | str) -> dict[str, Any]:
    """``{"header", "manifest", "tensors"}`` (tensors as fp32 arrays); every inconsistency is an error."""
    raw = Path(path).read_bytes()
    if len(raw) < HEADER_SIZE:
        raise ValueError(f"CSWG file too small: {len(raw)} bytes, need {HEADER_SIZE}")
    magic, version, dtype_code, n_manifest, reserved = _HEADER.unpack(raw[:HEADER_SIZE])
    if magic != MAGIC:
        raise ValueError(f"bad CSWG magic: expected {MAGIC!r}, got {magic!r}")
    if version != VERSION:
        raise ValueError(f"unsupported CSWG version: expected {VERSION}, got {version}")
    if dtype_code != DTYPE_FP16:
        raise ValueError(f"unsupported dtype code: expected {DTYPE_FP16} (fp16), got {dtype_code}")
    end = HEADER_SIZE + int(n_manifest)
    if end > len(raw):
        raise ValueError(f"CSWG manifest truncated: header says {n_manifest} bytes, file has {len(raw) - HEADER_SIZE}")
    manifest = json.loads(raw[HEADER_SIZE:end].decode())
    if int(manifest.get("version", -1)) != VERSION:
        raise ValueError("CSWG manifest version does not match header")
    payload = raw[end:]
    tensors: dict[str, np.ndarray] = {}
    for e in manifest["tensors"]:
        lo, n = int(e["offset"]), int(e["nbytes"])
        if lo + n > len(payload):
            raise ValueError(f"CSWG payload truncated reading {e['name']!r}: need bytes [{lo}, {lo + n}), "
                             f"payload has {len(payload)}")
        arr = np.frombuffer(payload[lo:lo + n], dtype=np.float16).astype(np.float32)
        tensors[str(e["name"])] = arr.reshape(tuple(int(x) for x in e["shape"]))
    used = max((int(e["offset"]) + int(e["nbytes"]) for e in manifest["tensors"]), default=0)
    if used != len(payload):
        raise ValueError(f"CSWG file has trailing payload bytes: manifest ends at {used}, payload_size={len(payload)}")
    return {"header": {"magic": "CSWG", "version": int(version), "dtype_code": int(dtype_code),
                       "manifest_bytes": int(n_manifest), "reserved": int(reserved)},
            "manifest": manifest, "tensors": tensors}


# ---------------------------------------------------------------------------
# native policy <-> named tensors
# ---------------------------------------------------------------------------
_BASE = ("W_vp", "b_vp", "W_lh", "b_lh", "W_sb", "alpha")
_BRANCH = ("lambda_hxh", "W_q", "W_k", "W_v", "W_o", "W_e")


def _dims_of(policy) -> dict[str, int]:
    return {"n_vertices": int(policy.N), "k_v": int(policy.K_v), "k_e": int(getattr(policy, "K_e", 1)),
            "k_s": int(policy.K_s), "h": int(policy.H), "n_heads": int(getattr(policy, "n_heads", 0)),
            "n_buckets": int(getattr(policy, "n_buckets", 0)), "bucket_embed_dim": int(getattr(policy, "embed_dim", 0))}


def policy_to_cswg(policy, path: Path | str) -> dict[str, Any]:
    dims = _dims_of(policy)
    shapes = tensor_shapes(dims)
    flat = np.asarray(policy.flat, np.float32)
    tensors: dict[str, np.ndarray] = {n: np.zeros(shapes[n], np.float32) for n in TENSOR_NAMES}
    o = 0
    order = _BASE + (_BRANCH if dims["n_heads"] > 0 else ()) + ("bucket_embed",)
    for name in order:
        n = int(np.prod(shapes[name], dtype=np.int64))
        tensors[name] = flat[o:o + n].reshape(shapes[name]).copy()
        o += n
    if o != flat.size:
        raise ValueError(f"policy carries {flat.size} weights, its dimensions describe {o}")
    tensors["temperature"] = np.float32(policy.temperature)
    return write_cswg_v3(path, tensors, dims)


def policy_from_cswg(path: Path | str):
    from . import native
    blob = load_cswg_v3(path)
    d, t = blob["manifest"]["dims"], blob["tensors"]
    plain = int(d["n_heads"]) == 0 and int(d["n_buckets"]) == 0 and int(d.get("k_e", 1)) == 1
    if plain:
        pol = native.SimplexPolicy(N=int(d["n_vertices"]), K_v=int(d["k_v"]), K_s=int(d["k_s"]), H=int(d["h"]))
    else:
        pol = native.SimplexPolicyV3(N=int(d["n_vertices"]), K_v=int(d["k_v"]), K_e=int(d["k_e"]), K_s=int(d["k_s"]),
                                     H=int(d["h"]), n_heads=int(d["n_heads"]), n_buckets=int(d["n_buckets"]),
                                     embed_dim=int(d["bucket_embed_dim"]))
    order = _BASE + (_BRANCH if int(d["n_heads"]) > 0 else ()) + (() if plain else ("bucket_embed",))
    flat = np.concatenate([np.asarray(t[n], np.float32).reshape(-1) for n in order]) if order else np.zeros(0, np.float32)
    if flat.size != pol.flat.size:
        raise ValueError(f"{path}: {flat.size} weights do not fit a policy of {pol.flat.size}")
    pol.flat = flat.astype(np.float32)
    pol.temperature = float(np.asarray(t["temperature"]).reshape(-1)[0])
    return pol
