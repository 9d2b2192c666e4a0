"""Reading and writing the safetensors container by tensor name.

Layout of a file: 8 bytes little-endian header length, a JSON header
{name: {dtype, shape, data_offsets}}, then the raw tensor bytes.  Files are
memory-mapped, so a tensor is only paged in when it is copied to the device.
A folder may hold one `model.safetensors` or shards listed in
`model.safetensors.index.json`.

The reference reads its own container the same way: one mmap, tensors by name,
an error that names the tensor that is missing (crates/quant/src/gguf.rs:228,
370, 466; crates/quant/src/error.rs:27).
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

_DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped .safetensors file."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.is_file():
            raise SafetensorsError(f"{self.path}: no such file")
        self._fh = open(self.path, "rb")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(self._fh.read(hlen))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{self.path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries = header
        self._base = 8 + hlen
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        for name, e in header.items():
            lo, hi = e["data_offsets"]
            if e["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has unsupported dtype {e['dtype']}")
            n = 1
            for d in e["shape"]:
                n *= d
            if hi - lo != n * _DTYPES[e["dtype"]].itemsize or self._base + hi > size:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has inconsistent offsets")

    def names(self):
        return list(self.entries)

    def shape(self, name):
        return tuple(self.entries[name]["shape"])

    def dtype(self, name):
        return _DTYPES[self.entries[name]["dtype"]]

    def tensor(self, name) -> torch.Tensor:
        """A CPU tensor that views the mapped bytes (read-only: copy before writing)."""
        e = self.entries[name]
        lo, hi = e["data_offsets"]
        dt = _DTYPES[e["dtype"]]
        if hi == lo:
            return torch.empty(tuple(e["shape"]), dtype=dt)
        buf = memoryview(self._mm)[self._base + lo: self._base + hi]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # torch warns that the buffer is not writable
            t = torch.frombuffer(buf, dtype=dt)
        return t.reshape(tuple(e["shape"]))

    def close(self):
        # views handed out by tensor() keep the map alive; dropping our handles is enough
        self._mm = None
        self._fh.close()


class ModelFiles:
    """All tensors of a model folder, whichever file holds them."""

    def __init__(self, folder):
        folder = Path(folder)
        index = folder / "model.safetensors.index.json"
        self.files: list[SafetensorsFile] = []
        self.where: dict[str, SafetensorsFile] = {}
        if index.is_file():
            wm = json.loads(index.read_text()).get("weight_map", {})
            opened: dict[str, SafetensorsFile] = {}
            for name, fname in wm.items():
                if fname not in opened:
                    opened[fname] = SafetensorsFile(folder / fname)
                    self.files.append(opened[fname])
                if name not in opened[fname].entries:
                    raise SafetensorsError(f"{index}: '{name}' is not in {fname}")
                self.where[name] = opened[fname]
        else:
            f = SafetensorsFile(folder / "model.safetensors")
            self.files.append(f)
            self.where = {n: f for n in f.names()}

    def names(self):
        return list(self.where)

    def shape(self, name):
        return self.where[name].shape(name)

    def dtype(self, name):
        return self.where[name].dtype(name)

    def tensor(self, name):
        return self.where[name].tensor(name)

    def close(self):
        for f in self.files:
            f.close()


def write_safetensors(path, tensors: dict, metadata: dict | None = None) -> None:
    """Write CPU tensors under their names; offsets are 8-byte aligned by
    padding the header with spaces, as the format allows."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            fh.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
