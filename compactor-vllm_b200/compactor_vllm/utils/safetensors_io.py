"""Reader for .safetensors files: an 8-byte little-endian header length, that many bytes of JSON
(name -> dtype, shape, data_offsets), then the raw little-endian data.  Tensors are returned as torch CPU tensors
that view a memory map of the file; nothing is copied until a caller moves them."""
from __future__ import annotations

import json
import struct
from typing import Dict

import numpy as np
import torch

_DTYPES = {
    "F32": (np.dtype("<f4"), torch.float32), "F16": (np.dtype("<f2"), torch.float16),
    "BF16": (np.dtype("<i2"), torch.bfloat16), "F64": (np.dtype("<f8"), torch.float64),
    "I64": (np.dtype("<i8"), torch.int64), "I32": (np.dtype("<i4"), torch.int32),
    "I16": (np.dtype("<i2"), torch.int16), "I8": (np.dtype("i1"), torch.int8),
    "U8": (np.dtype("u1"), torch.uint8), "BOOL": (np.dtype("u1"), torch.bool),
}


def load_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    base = 8 + n
    data = np.memmap(path, dtype=np.uint8, mode="r")
    out: Dict[str, torch.Tensor] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if meta["dtype"] not in _DTYPES:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {meta['dtype']}")
        np_dt, th_dt = _DTYPES[meta["dtype"]]
        lo, hi = meta["data_offsets"]
        shape = tuple(int(x) for x in meta["shape"])
        count = int(np.prod(shape)) if shape else 1
        if hi - lo != count * np_dt.itemsize:
            raise ValueError(f"{path}: tensor {name} has {hi - lo} bytes for shape {shape}")
        arr = np.frombuffer(data, dtype=np_dt, count=count, offset=base + lo)
        t = torch.from_numpy(arr.copy())         # the map is read-only; a copy also frees it early
        if th_dt is torch.bfloat16:
            t = t.view(torch.bfloat16)
        elif th_dt is torch.bool:
            t = t.to(torch.bool)
        out[name] = t.reshape(shape)
    return out
