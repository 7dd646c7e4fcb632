"""Minimal reader / writer of the safetensors container, enough for checkpoints of the models served here.

Layout of a file: an 8-byte little-endian header length, that many bytes of JSON (``name -> {dtype, shape,
data_offsets}``, plus an optional ``__metadata__`` entry), then the raw little-endian tensor data.  Reading maps
the file and copies each tensor out, so nothing but torch and the standard library is needed.
"""
from __future__ import annotations

import json
import mmap
import struct
from typing import Dict

import torch

_DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of a file, on the CPU, in their stored dtypes."""
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file")
        (n,) = struct.unpack("<Q", head)
        header = json.loads(f.read(n).decode("utf-8"))
        base = 8 + n
        with mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) as mm:
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                try:
                    dtype = _DTYPES[meta["dtype"]]
                except KeyError:
                    raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {meta['dtype']!r}") from None
                lo, hi = meta["data_offsets"]
                shape = [int(d) for d in meta["shape"]]
                count = 1
                for d in shape:
                    count *= d
                if hi - lo != count * torch.empty((), dtype=dtype).element_size():
                    raise ValueError(f"{path}: tensor {name!r} has {hi - lo} bytes, its shape says otherwise")
                raw = bytearray(mm[base + lo: base + hi])
                t = torch.frombuffer(raw, dtype=dtype) if count else torch.empty(0, dtype=dtype)
                out[name] = t.reshape(shape).clone()
    return out


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    header, blobs, at = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        data = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(data)]}
        blobs.append(data)
        at += len(data)
    head = json.dumps(header, separators=(",", ":")).encode("utf-8")
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
