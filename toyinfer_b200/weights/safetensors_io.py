"""Reader and writer for the safetensors container.

Format (the one the reference's export script scans, export.py:211-230 and
export.py:272-277, and its loader assumes, src/qwen.cpp:446-451): an 8-byte
little-endian header length N, N bytes of JSON mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end
of the header; the ``__metadata__`` key is not a tensor), then the raw
little-endian data.  Files are memory-mapped; a tensor is a zero-copy view until
the loader moves it to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "F32": torch.float32,
    "F64": torch.float64,
    "I32": torch.int32,
    "I64": torch.int64,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int  # absolute byte offset in the file
    end: int
    file: str


class SafetensorsFile:
    """One memory-mapped file; ``entries`` maps tensor name to its description."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a safetensors header")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds file size {size}")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not valid JSON ({exc})") from exc
        base = 8 + hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype = _DTYPES[meta["dtype"]]
            except KeyError:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} has unsupported dtype {meta.get('dtype')!r}"
                ) from None
            shape = tuple(int(s) for s in meta["shape"])
            b, e = (int(x) for x in meta["data_offsets"])
            count = 1
            for s in shape:
                count *= s
            want = count * torch.empty((), dtype=dtype).element_size()
            if e - b != want:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} spans {e - b} bytes but shape {shape} needs {want}"
                )
            if base + e > size:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} ends at byte {base + e} beyond the file's {size} (truncated?)"
                )
            self.entries[name] = TensorEntry(name, dtype, shape, base + b, base + e, path)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the tensor's bytes (no copy)."""
        e = self.entries[name]
        count = 1
        for s in e.shape:
            count *= s
        if count == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; nobody writes to the view
            flat = torch.frombuffer(self._mm, dtype=e.dtype, count=count, offset=e.begin)
        return flat.view(e.shape)

    def close(self) -> None:
        # Views handed out keep the map alive through the buffer protocol; closing
        # while views exist raises BufferError, which only means "still in use".
        try:
            if self._mm is not None:
                self._mm.close()
        except BufferError:
            pass
        self._f.close()


def model_files(model_dir: str) -> List[str]:
    """Shard paths of a model folder: the index's ``weight_map`` when there is one,
    otherwise every ``*.safetensors`` file in name order."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            wm = json.load(f).get("weight_map", {})
        names = sorted(set(wm.values()))
        files = [os.path.join(model_dir, n) for n in names]
    else:
        files = sorted(
            os.path.join(model_dir, n) for n in os.listdir(model_dir) if n.endswith(".safetensors")
        )
    if not files:
        raise SafetensorsError(f"{model_dir}: no .safetensors file found")
    for p in files:
        if not os.path.isfile(p):
            raise SafetensorsError(f"{p}: named by the index but not found")
    return files


def open_model(model_dir: str) -> Tuple[List[SafetensorsFile], Dict[str, SafetensorsFile]]:
    """Open every shard; returns the files and a map tensor name -> file."""
    files = [SafetensorsFile(p) for p in model_files(model_dir)]
    where: Dict[str, SafetensorsFile] = {}
    for f in files:
        for name in f.entries:
            if name in where:
                raise SafetensorsError(
                    f"tensor {name!r} is stored twice: in {where[name].path} and {f.path}"
                )
            where[name] = f
    return files, where


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Write tensors (name, CPU tensor) in the given order."""
    header = {}
    blobs = []
    offset = 0
    for name, t in tensors:
        t = t.detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of {name!r}")
        nbytes = t.numel() * t.element_size()
        header[name] = {
            "dtype": _NAMES[t.dtype],
            "shape": list(t.shape),
            "data_offsets": [offset, offset + nbytes],
        }
        blobs.append(t)
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t in blobs:
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().data)
