"""Reading and writing safetensors files without any library in between.

File format (the reference parses it by hand as well, model/export_safetensors.py:24-48):
8 bytes little-endian header length ``n``; ``n`` bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``;
then the raw little-endian tensor bytes, offsets relative to the end of the
header.  Sharded models carry ``model.safetensors.index.json`` whose
``weight_map`` maps each name to its shard (model/export_safetensors.py:51-60).

Tensors are returned as views of a memory map: nothing is copied until the
loader moves a tensor to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch


class WeightFileError(RuntimeError):
    """The file is not a readable safetensors file."""


_DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One .safetensors file, opened as a memory map."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise WeightFileError(f"cannot open {path}: {e.strerror}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise WeightFileError(f"{path}: {size} bytes is too short for a safetensors header")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if 8 + n > size:
            raise WeightFileError(f"{path}: header claims {n} bytes but the file has {size}")
        try:
            header = json.loads(self._f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise WeightFileError(f"{path}: header is not valid JSON ({e})") from None
        self._base = 8 + n
        self._size = size
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, dict] = {}
        for name, meta in header.items():
            dt = meta.get("dtype")
            if dt not in _DTYPES:
                raise WeightFileError(f"{path}: tensor '{name}' has unsupported dtype {dt!r}")
            b, e = meta["data_offsets"]
            numel = 1
            for s in meta["shape"]:
                numel *= s
            want = numel * torch.empty((), dtype=_DTYPES[dt]).element_size()
            if e - b != want:
                raise WeightFileError(f"{path}: tensor '{name}' spans {e - b} bytes, its shape needs {want}")
            if self._base + e > size:
                raise WeightFileError(f"{path}: tensor '{name}' ends at byte {self._base + e}, "
                                      f"the file has {size} (truncated?)")
            self.entries[name] = meta
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the tensor's bytes in the file."""
        meta = self.entries[name]
        b, e = meta["data_offsets"]
        dt = _DTYPES[meta["dtype"]]
        if e == b:
            return torch.empty(tuple(meta["shape"]), dtype=dt)
        buf = memoryview(self._mm)[self._base + b:self._base + e]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            t = torch.frombuffer(buf, dtype=dt)
        return t.reshape(tuple(meta["shape"]))

    def close(self) -> None:
        # views handed out keep the map alive; closing the file object is enough
        self._f.close()


def open_model_files(folder: str) -> Dict[str, SafetensorsFile]:
    """Open the weight files of a model folder; returns name -> file that holds it."""
    idx = os.path.join(folder, "model.safetensors.index.json")
    single = os.path.join(folder, "model.safetensors")
    by_name: Dict[str, SafetensorsFile] = {}
    if os.path.exists(idx):
        with open(idx, "r", encoding="utf-8") as f:
            weight_map = json.load(f).get("weight_map", {})
        files: Dict[str, SafetensorsFile] = {}
        for name, shard in weight_map.items():
            if shard not in files:
                files[shard] = SafetensorsFile(os.path.join(folder, shard))
            if name not in files[shard].entries:
                raise WeightFileError(f"{idx} places '{name}' in {shard}, which does not hold it")
            by_name[name] = files[shard]
        # tensors present in a shard but absent from the index are still reported
        for sf in files.values():
            for name in sf.names():
                by_name.setdefault(name, sf)
    elif os.path.exists(single):
        sf = SafetensorsFile(single)
        for name in sf.names():
            by_name[name] = sf
    else:
        raise WeightFileError(f"{folder} holds neither model.safetensors nor model.safetensors.index.json")
    return by_name


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata=None, layout=None) -> None:
    """Write tensors in the order given.  ``layout``: a list of ``(name, dtype, shape)`` in that order; with
    it the header is written first and the tensors are taken from the iterable and written one at a time,
    so that a large model is never held in memory as a whole.  Without it the tensors are collected first."""
    if layout is None:
        tensors = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
        layout = [(n, t.dtype, tuple(t.shape)) for n, t in tensors]
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for name, dt, shape in layout:
        if dt not in _NAMES:
            raise WeightFileError(f"cannot store dtype {dt} of '{name}'")
        numel = 1
        for d in shape:
            numel *= int(d)
        nbytes = numel * torch.empty((), dtype=dt).element_size()
        header[name] = {"dtype": _NAMES[dt], "shape": [int(d) for d in shape], "data_offsets": [off, off + nbytes]}
        off += nbytes
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        it = iter(tensors)
        for name, dt, shape in layout:
            try:
                got_name, t = next(it)
            except StopIteration:
                raise WeightFileError(f"the tensors end before '{name}'") from None
            t = t.detach().cpu().contiguous()
            if got_name != name or t.dtype != dt or tuple(t.shape) != tuple(shape):
                raise WeightFileError(f"expected '{name}' {dt} {list(shape)}, got '{got_name}' {t.dtype} {list(t.shape)}")
            if t.numel():
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)
