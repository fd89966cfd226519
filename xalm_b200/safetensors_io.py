"""Reader and writer for model folders described by a config.json: `config.json` + `model.safetensors`.

A safetensors file is an 8-byte little-endian header length, that many bytes of JSON (name -> dtype, shape,
data_offsets relative to the end of the header), then the payloads.  Only what the backend uploads is handled:
F32 / F16 / BF16 matrices and vectors; integer tables are passed through as raw bytes.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np

from . import types as T

_DTYPES = {"F32": (T.F32, 4), "F16": (T.F16, 2), "BF16": (T.BF16, 2)}
_RAW = {"I32": 4, "I64": 8, "U8": 1}


def read_header(path: str):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    header.pop("__metadata__", None)
    return header, 8 + n


def read_tensors(path: str) -> "dict[str, tuple[T.XType | None, tuple, np.ndarray]]":
    """name -> (type, shape, raw payload as uint8); type is None for integer tables."""
    header, base = read_header(path)
    data = np.fromfile(path, dtype=np.uint8)
    out = {}
    for name, info in header.items():
        lo, hi = info["data_offsets"]
        raw = data[base + lo: base + hi]
        dt = info["dtype"]
        if dt in _DTYPES:
            t, esz = _DTYPES[dt]
        elif dt in _RAW:
            t, esz = None, _RAW[dt]
        else:
            raise ValueError(f"{path}: tensor {name} has dtype {dt} (F32, F16, BF16 or an integer table)")
        if raw.size != int(np.prod(info["shape"], dtype=np.int64)) * esz:
            raise ValueError(f"{path}: tensor {name}: {raw.size} bytes for shape {info['shape']}")
        out[name] = (t, tuple(info["shape"]), raw)
    return out


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def write_model_dir(path: str, config: dict, tensors: "dict[str, np.ndarray]", dtype: str = "BF16") -> None:
    """Write config.json and model.safetensors; float arrays are stored as `dtype` (BF16, F16 or F32)."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    header, blobs, at = {}, [], 0
    for name, a in tensors.items():
        a = np.asarray(a)
        if dtype == "BF16":
            raw = f32_to_bf16_bits(a).tobytes()
        elif dtype == "F16":
            raw = a.astype(np.float16).tobytes()
        else:
            raw = a.astype(np.float32).tobytes()
        header[name] = {"dtype": dtype, "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
