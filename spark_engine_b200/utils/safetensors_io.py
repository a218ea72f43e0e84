"""safetensors files: a small writer (tests, shard tools) and a loader on top of the C++ reader.

Format: 8-byte little-endian header length, JSON header {name: {dtype, shape, data_offsets}}, raw bytes.
Reference: engine-rs/src/safetensors.rs; per-rank pre-split shard files (ds41/shard.rs:1-116) are written with
`write_safetensors` by `shard_tool`.
"""
from __future__ import annotations

import json
import struct
from typing import Dict

import torch

from ..runtime import rt

_DT = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int16: "I16", torch.int32: "I32",
       torch.int64: "I64", torch.uint8: "U8", torch.int8: "I8", torch.float8_e4m3fn: "F8_E4M3"}
_RDT = {v: k for k, v in _DT.items()}


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    header, off, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = metadata
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _DT[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def load_safetensors(path: str, device="cpu", pinned_staging: bool = False) -> Dict[str, torch.Tensor]:
    """Every tensor of a file.  With `pinned_staging` each tensor is pread into pinned memory and copied to the
    device asynchronously (the fast-load path of the reference: pread -> pinned staging -> device)."""
    st = rt().SafeTensors(path)
    out = {}
    for name in st.names():
        info = st.info(name)
        dt = _RDT[info.dtype]
        n = info.end - info.begin
        buf = torch.empty(n, dtype=torch.uint8, pin_memory=pinned_staging and torch.cuda.is_available())
        if n:
            st.read_into(name, buf.data_ptr(), n)
        t = buf.view(dt).view(*info.shape) if n else torch.empty(*info.shape, dtype=dt)
        out[name] = t.to(device, non_blocking=pinned_staging)
    return out
