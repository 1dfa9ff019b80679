"""Reader of safetensors checkpoints: an 8-byte little-endian header length, that many bytes of JSON
(name -> dtype, shape, data_offsets), then the raw little-endian data.  Tensors come back as CPU torch tensors in
their stored type; nothing but the standard library, numpy and torch is used."""
from __future__ import annotations

import json
import struct

import numpy as np
import torch

_NP = {"F32": np.float32, "F16": np.float16, "I32": np.int32, "I64": np.int64, "I8": np.int8, "U8": np.uint8}


def read_safetensors(path: str) -> dict:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        index = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in index.items():
        if name == "__metadata__":
            continue
        lo, hi = e["data_offsets"]
        raw, shape = data[lo:hi], tuple(e["shape"])
        if e["dtype"] == "BF16":
            t = torch.from_numpy(np.frombuffer(raw, dtype=np.int16).copy()).view(torch.bfloat16)
        elif e["dtype"] in _NP:
            t = torch.from_numpy(np.frombuffer(raw, dtype=_NP[e["dtype"]]).copy())
        else:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {e['dtype']}")
        out[name] = t.reshape(shape)
    return out


def write_safetensors(path: str, tensors: dict) -> None:
    """The inverse (tests and examples write small random checkpoints with it)."""
    names = {torch.bfloat16: "BF16", torch.float32: "F32", torch.float16: "F16", torch.int32: "I32", torch.int64: "I64"}
    index, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        index[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hdr = json.dumps(index).encode()
    hdr += b" " * (-len(hdr) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"".join(blobs))
