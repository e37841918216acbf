"""Reading and writing safetensors files without a third-party package: 8 bytes little-endian header length, a JSON header
(name -> dtype, shape, data_offsets into the byte buffer that follows), then the tensors' bytes."""
from __future__ import annotations

import json
import struct
from typing import Dict

import numpy as np
import torch

_DTYPES = {"BF16": (torch.bfloat16, 2), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "I32": (torch.int32, 4), "I64": (torch.int64, 8)}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


def load_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        if n > (1 << 30):
            raise ValueError(f"{path}: implausible header length {n}")
        header = json.loads(f.read(n))
        data = f.read()
    out: Dict[str, torch.Tensor] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if meta["dtype"] not in _DTYPES:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {meta['dtype']}")
        dt, size = _DTYPES[meta["dtype"]]
        a, b = meta["data_offsets"]
        count = 1
        for s in meta["shape"]:
            count *= int(s)
        if b - a != count * size or b > len(data):
            raise ValueError(f"{path}: tensor {name} does not fit its byte range")
        raw = np.frombuffer(data, dtype=np.uint8, count=b - a, offset=a).copy()
        out[name] = torch.from_numpy(raw).view(dt).reshape(meta["shape"])
    return out


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
