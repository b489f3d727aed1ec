"""Reader and writer for the safetensors container, by tensor name.

Format (as the reference parses it, ``pkg/model/loader.go:173-232``): an 8-byte
little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the
header; the key ``__metadata__`` is skipped), then the raw little-endian data.  A model is
either one ``model.safetensors`` or shards listed by ``model.safetensors.index.json``'s
``weight_map`` (``pkg/model/loader.go:128-170``).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Tuple

import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 << 20   # a header larger than this is a corrupt file, not a model


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    file: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int      # absolute byte offsets in the file
    end: int


def read_header(path: str) -> Dict[str, TensorEntry]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) < 8:
            raise SafetensorsError(f"{path}: shorter than its 8-byte header length")
        (hlen,) = struct.unpack("<Q", raw)
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} is not plausible for a {size}-byte file")
        try:
            header = json.loads(f.read(hlen))
        except ValueError as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
    base = 8 + hlen
    out: Dict[str, TensorEntry] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dt = meta.get("dtype")
        if dt not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
        tdt, isz = _DTYPES[dt]
        shape = tuple(int(s) for s in meta["shape"])
        b, e = meta["data_offsets"]
        n = 1
        for s in shape:
            n *= s
        if e - b != n * isz or base + e > size or b < 0:
            raise SafetensorsError(f"{path}: tensor {name!r} of shape {shape} {dt} does not fit its "
                                   f"data_offsets [{b}, {e}]")
        out[name] = TensorEntry(path, tdt, shape, base + b, base + e)
    return out


def index_model_dir(model_dir: str) -> Dict[str, TensorEntry]:
    """Name -> entry for every tensor of the model folder (single file or shards)."""
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(idx):
        with open(idx) as f:
            wm = json.load(f).get("weight_map", {})
        entries: Dict[str, TensorEntry] = {}
        for shard in sorted(set(wm.values())):
            entries.update(read_header(os.path.join(model_dir, shard)))
        return entries
    if os.path.isfile(single):
        return read_header(single)
    raise SafetensorsError(f"no model.safetensors (or model.safetensors.index.json) in {model_dir}")


class MappedFiles:
    """Memory maps of the files behind a set of entries; tensors are copied out of the map."""

    def __init__(self):
        self._maps: Dict[str, mmap.mmap] = {}

    def read(self, e: TensorEntry) -> torch.Tensor:
        m = self._maps.get(e.file)
        if m is None:
            with open(e.file, "rb") as f:
                m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps[e.file] = m
        n = 1
        for s in e.shape:
            n *= s
        if n == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # read-only map: the tensor is copied at once
            t = torch.frombuffer(m, dtype=e.dtype, count=n, offset=e.begin)
        return t.reshape(e.shape).clone()

    def close(self):
        for m in self._maps.values():
            try:
                m.close()
            except BufferError:
                pass
        self._maps.clear()


def write_file(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) as one safetensors file, names sorted."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
