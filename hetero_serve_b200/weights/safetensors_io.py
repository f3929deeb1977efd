"""A small reader and writer for the safetensors container.

Layout of a file: an unsigned 64-bit little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``
and the raw little-endian tensor bytes.  The reference parses the same container
by hand into 32-bit numpy arrays (heteroserve/model/fetch.py:74-119), widening
bfloat16 on the way; this reader keeps every tensor in the type it was stored
in (bfloat16 stays bfloat16, 32-bit stays 32-bit) and narrows integer tensors to
int32, the width the kernels index with.
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
    "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
    "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_TAGS = {v: k for k, v in _DTYPES.items()}
_INTEGER = {torch.int64, torch.int16, torch.int8, torch.uint8}
_HEADER_LIMIT = 100 * 1024 * 1024


class SafetensorsError(ValueError):
    pass


def read_header(path: str | Path) -> tuple[dict, int]:
    """Return ``(header without __metadata__, offset of the data section)``."""
    path = Path(path)
    size = path.stat().st_size
    with open(path, "rb") as fh:
        head = fh.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors file")
        (n,) = struct.unpack("<Q", head)
        if n > _HEADER_LIMIT or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file")
        try:
            header = json.loads(fh.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not JSON ({exc})") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header is not a JSON object")
    header.pop("__metadata__", None)
    return header, 8 + n


def read_safetensors(path: str | Path) -> dict[str, torch.Tensor]:
    """Read every tensor of a file, each in its stored type (integers → int32)."""
    path = Path(path)
    header, data_start = read_header(path)
    out: dict[str, torch.Tensor] = {}
    with open(path, "rb") as fh:
        size = path.stat().st_size
        if size == data_start:
            blob = b""
        else:
            blob = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_COPY)
        for name, meta in header.items():
            try:
                tag, shape = meta["dtype"], [int(s) for s in meta["shape"]]
                begin, end = (int(x) for x in meta["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for {name!r}") from None
            dtype = _DTYPES.get(tag)
            if dtype is None:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {tag}")
            count = 1
            for s in shape:
                count *= s
            itemsize = torch.empty((), dtype=dtype).element_size()
            if end - begin != count * itemsize or begin < 0 or data_start + end > size:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} of shape {shape} and dtype {tag} does not "
                    f"match its byte range [{begin}, {end})")
            if count == 0:
                t = torch.empty(shape, dtype=dtype)
            else:
                t = torch.frombuffer(blob, dtype=dtype, count=count,
                                     offset=data_start + begin).reshape(shape).clone()
            if dtype in _INTEGER:
                t = t.to(torch.int32)
            out[name] = t
        if blob:
            blob.close()
    return out


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor],
                      metadata: dict[str, str] | None = None) -> None:
    """Write tensors (on the CPU, any supported type) in name order."""
    path = Path(path)
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TAGS:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _TAGS[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + n]}
        offset += n
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(raw)))
        fh.write(raw)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                fh.write(t.view(torch.uint8).numpy().tobytes()
                         if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
