"""Reader and writer of the safetensors container, written from its layout:
8 bytes of little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}``, then the data.

The header is validated exhaustively before any byte of data is trusted, in the
manner of the reference's parser (src/formats.rs:1186-1333): short file, header
length beyond the file, header that is no JSON object, unknown dtype, offsets
outside the data, a span that does not equal shape x dtype size, overlapping
spans.  Shards are found through ``model.safetensors.index.json``
(src/formats.rs:1458-1518); a tensor in two shards is an error.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

_DTYPES = {
    # name: (bytes per element, numpy dtype used to view the bytes, torch dtype of the view)
    "F64": (8, np.float64, torch.float64),
    "F32": (4, np.float32, torch.float32),
    "F16": (2, np.float16, torch.float16),
    "BF16": (2, np.uint16, torch.bfloat16),
    "I64": (8, np.int64, torch.int64),
    "I32": (4, np.int32, torch.int32),
    "I16": (2, np.int16, torch.int16),
    "I8": (1, np.int8, torch.int8),
    "U8": (1, np.uint8, torch.uint8),
    "BOOL": (1, np.uint8, torch.bool),
}
_TORCH_TO_NAME = {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16",
                  torch.bfloat16: "BF16", torch.int64: "I64", torch.int32: "I32",
                  torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL"}
_MAX_HEADER = 100 << 20


class SafetensorsError(ValueError):
    pass


def parse_header(buf, path: str) -> Tuple[Dict[str, dict], int]:
    """({tensor name: {"dtype", "shape", "begin", "end"}}, offset of the data)."""
    size = len(buf)
    if size < 8:
        raise SafetensorsError(f"{path}: file of {size} bytes is too short for a safetensors header")
    (hlen,) = struct.unpack("<Q", buf[:8])
    if hlen > size - 8 or hlen > _MAX_HEADER:
        raise SafetensorsError(f"{path}: header length {hlen} exceeds the file ({size} bytes)")
    try:
        header = json.loads(bytes(buf[8:8 + hlen]).decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header is not a JSON object")
    data_len = size - 8 - hlen
    out: Dict[str, dict] = {}
    spans: List[Tuple[int, int, str]] = []
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if not isinstance(meta, dict):
            raise SafetensorsError(f"{path}: entry '{name}' is not an object")
        dtype, shape, offs = meta.get("dtype"), meta.get("shape"), meta.get("data_offsets")
        if dtype not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dtype!r}")
        if not isinstance(shape, list) or any(isinstance(s, bool) or not isinstance(s, int) or s < 0 for s in shape):
            raise SafetensorsError(f"{path}: tensor '{name}' has a malformed shape {shape!r}")
        if (not isinstance(offs, list) or len(offs) != 2
                or any(isinstance(o, bool) or not isinstance(o, int) for o in offs)):
            raise SafetensorsError(f"{path}: tensor '{name}' has malformed data_offsets {offs!r}")
        begin, end = offs
        if begin < 0 or end < begin or end > data_len:
            raise SafetensorsError(f"{path}: tensor '{name}' spans [{begin}, {end}) outside the data "
                                   f"({data_len} bytes)")
        n = 1
        for s in shape:
            n *= s
        if n * _DTYPES[dtype][0] != end - begin:
            raise SafetensorsError(f"{path}: tensor '{name}' of shape {shape} and dtype {dtype} needs "
                                   f"{n * _DTYPES[dtype][0]} bytes but spans {end - begin}")
        out[name] = {"dtype": dtype, "shape": tuple(shape), "begin": begin, "end": end}
        if end > begin:
            spans.append((begin, end, name))
    spans.sort()
    for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
        if b1 < e0:
            raise SafetensorsError(f"{path}: tensors '{n0}' and '{n1}' overlap in the data")
    return out, 8 + hlen


class SafetensorsFile:
    """One mapped file; tensors are views of the mapping until copied."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e}") from e
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            self._f.close()
            raise SafetensorsError(f"{path}: file of {size} bytes is too short for a safetensors header")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.tensors, self._data0 = parse_header(self._map, path)

    def names(self) -> Iterable[str]:
        return self.tensors.keys()

    def read(self, name: str) -> torch.Tensor:
        """A copy of the tensor in its stored dtype."""
        meta = self.tensors[name]
        nbytes, np_dtype, t_dtype = _DTYPES[meta["dtype"]]
        count = (meta["end"] - meta["begin"]) // nbytes
        if count == 0:
            return torch.empty(meta["shape"], dtype=t_dtype)
        arr = np.frombuffer(self._map, dtype=np_dtype, count=count, offset=self._data0 + meta["begin"])
        t = torch.from_numpy(arr.copy())
        if t_dtype is torch.bfloat16:
            t = t.view(torch.bfloat16)
        elif t_dtype is torch.bool:
            t = t.to(torch.bool)
        return t.reshape(meta["shape"])

    def close(self) -> None:
        try:
            self._map.close()
        finally:
            self._f.close()


def open_model_files(folder: str) -> Dict[str, Tuple[SafetensorsFile, str]]:
    """{tensor name: (file, name)} over ``model.safetensors`` or the shards of its index."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    files: List[str] = []
    if os.path.exists(single):
        files = [single]
    elif os.path.exists(index):
        try:
            with open(index) as f:
                wm = json.load(f)["weight_map"]
        except (OSError, KeyError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{index}: cannot read the weight_map: {e}") from e
        for shard in sorted(set(wm.values())):
            p = os.path.join(folder, shard)
            if not os.path.exists(p):
                raise SafetensorsError(f"{index} names shard '{shard}', which does not exist")
            files.append(p)
    else:
        raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json found")
    where: Dict[str, Tuple[SafetensorsFile, str]] = {}
    for p in files:
        sf = SafetensorsFile(p)
        for n in sf.names():
            if n in where:
                raise SafetensorsError(f"tensor '{n}' appears in both {where[n][0].path} and {p}")
            where[n] = (sf, n)
    return where


def _raw_bytes(t: torch.Tensor) -> memoryview:
    flat = t.detach().cpu().contiguous().reshape(-1)
    if flat.dtype is torch.bool:
        flat = flat.to(torch.uint8)
    return memoryview(flat.view(torch.uint8).numpy())


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    """Write tensors in name order; the header is padded so that the data starts 8-byte aligned."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"tensor '{name}' has dtype {t.dtype}, which safetensors cannot hold")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for name in order:
            f.write(_raw_bytes(tensors[name]))
    os.replace(tmp, path)
