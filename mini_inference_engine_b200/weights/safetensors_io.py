"""Reading and writing the safetensors container: an 8-byte little-endian header length,
a JSON header ``{name: {dtype, shape, data_offsets}}`` and the raw little-endian data.
The reference reads the same files through the safetensors package
(inference_engine/weights.py:15-21); this reader maps the file instead of copying it and
needs nothing beyond torch."""
from __future__ import annotations

import json
import mmap
import os
import struct

import torch

_DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def read_header(path: str) -> tuple[dict, int]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        if n > size - 8:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file")
        try:
            header = json.loads(f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
    return header, 8 + n


def read_file(path: str) -> dict[str, torch.Tensor]:
    """All tensors of one file, as views of a read-only mapping (copy before writing)."""
    header, base = read_header(path)
    out: dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        if os.path.getsize(path) == base:
            return out
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)   # private pages: torch may not write through
    for name, info in header.items():
        if name == "__metadata__":
            continue
        try:
            dt = _DTYPES[info["dtype"]]
        except KeyError:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {info.get('dtype')!r}") from None
        shape = tuple(info["shape"])
        b, e = info["data_offsets"]
        numel = 1
        for s in shape:
            numel *= s
        if e - b != numel * torch.empty((), dtype=dt).element_size():
            raise SafetensorsError(f"{path}: tensor {name!r}: {e - b} bytes do not hold shape {shape} of {info['dtype']}")
        if numel == 0:
            out[name] = torch.empty(shape, dtype=dt)
            continue
        out[name] = torch.frombuffer(mm, dtype=dt, count=numel, offset=base + b).view(shape)
    return out


def write_file(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} (tensor {name!r})")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * (-len(hb) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
