"""Reader and writer of safetensors files and the bfloat16 <-> float32 conversions the model loaders share.

A file is an 8-byte little-endian header length, that many bytes of JSON (name -> dtype, shape, data_offsets), then the data."""
from __future__ import annotations

import json
import struct

import numpy as np

from .capi import TensorError


def bf16_to_f32(u16: np.ndarray) -> np.ndarray:
    return (u16.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """round to nearest even, as uint16 bit patterns"""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def read_safetensors(path: str) -> dict:
    """-> ({name: ndarray}, names stored as bfloat16); bfloat16 tensors come back as their uint16 bit patterns."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(n))
        data = f.read()
    kinds = {"BF16": np.uint16, "F32": np.float32, "F16": np.float16, "I32": np.int32}
    out, bf16 = {}, set()
    for name, m in meta.items():
        if name == "__metadata__":
            continue
        if m["dtype"] not in kinds:
            raise TensorError(f"{name}: unsupported dtype {m['dtype']}")
        a, b = m["data_offsets"]
        out[name] = np.frombuffer(data[a:b], kinds[m["dtype"]]).reshape(m["shape"])
        if m["dtype"] == "BF16":
            bf16.add(name)
    return out, bf16


def write_safetensors(path: str, tensors: dict):
    """tensors: {name: float32 ndarray}; stored as bfloat16 (used by tests and examples to make model folders)."""
    meta, blobs, off = {}, [], 0
    for name, a in tensors.items():
        raw = f32_to_bf16(np.asarray(a, np.float32)).tobytes()
        meta[name] = {"dtype": "BF16", "shape": list(np.asarray(a).shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hdr = json.dumps(meta).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"".join(blobs))


