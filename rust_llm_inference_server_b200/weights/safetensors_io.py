"""Reader and writer for the safetensors container: an 8-byte little-endian header length, a JSON
header {name: {dtype, shape, data_offsets}}, then the raw little-endian tensor bytes.

The reference maps every `*.safetensors` file of the model folder, sorted, into one name space
(crates/model/src/llama.rs:126-137); `open_model_dir` does the same.
"""

from __future__ import annotations

import glob
import json
import os
import struct

import numpy as np
import torch

# safetensors dtype tag -> (torch dtype, numpy storage dtype)
_DTYPES = {
    "F64": (torch.float64, np.float64), "F32": (torch.float32, np.float32),
    "F16": (torch.float16, np.float16), "BF16": (torch.bfloat16, np.uint16),
    "I64": (torch.int64, np.int64), "I32": (torch.int32, np.int32),
    "I16": (torch.int16, np.int16), "I8": (torch.int8, np.int8),
    "U8": (torch.uint8, np.uint8), "BOOL": (torch.bool, np.bool_),
}
_TAG_OF = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped file; tensors are views into the map until they are copied."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise SafetensorsError(f"{path}: too short to be a safetensors file")
            (n,) = struct.unpack("<Q", head)
            if n <= 0 or 8 + n > size:
                raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
            try:
                header = json.loads(f.read(n).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{path}: header is not JSON: {e}") from e
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: dict[str, dict] = header
        self._data_start = 8 + n
        self._map = None
        for name, e in header.items():
            if e.get("dtype") not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name}: element type {e.get('dtype')!r} is not known")
            b, en = e["data_offsets"]
            count = int(np.prod(e["shape"])) if e["shape"] else 1
            width = np.dtype(_DTYPES[e["dtype"]][1]).itemsize
            if en - b != count * width or self._data_start + en > size:
                raise SafetensorsError(f"{path}: tensor {name}: offsets {b}..{en} do not match shape "
                                       f"{e['shape']} of {e['dtype']}")

    def names(self):
        return list(self.entries)

    def shape(self, name: str) -> tuple:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]][0]

    def get(self, name: str) -> torch.Tensor:
        """The tensor as stored (its own element type), on the CPU, backed by the file map."""
        e = self.entries[name]
        tdt, ndt = _DTYPES[e["dtype"]]
        if self._map is None:
            # copy-on-write map: pages are read lazily and nothing is ever written back
            self._map = np.memmap(self.path, dtype=np.uint8, mode="c")
        b, en = e["data_offsets"]
        raw = self._map[self._data_start + b:self._data_start + en]
        arr = raw.view(ndt).reshape(e["shape"])
        t = torch.from_numpy(arr)
        return t.view(torch.bfloat16) if tdt == torch.bfloat16 else t


class Checkpoint:
    """Tensors by name over one or several files (or an in-memory dictionary)."""

    def __init__(self, files: list[SafetensorsFile] | None = None, tensors: dict | None = None):
        self._where: dict[str, SafetensorsFile] = {}
        self._mem: dict[str, torch.Tensor] = dict(tensors or {})
        for f in files or []:
            for n in f.names():
                self._where[n] = f

    def names(self) -> list[str]:
        return sorted(set(self._where) | set(self._mem))

    def shape(self, name: str) -> tuple:
        return tuple(self._mem[name].shape) if name in self._mem else self._where[name].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._mem[name].dtype if name in self._mem else self._where[name].dtype(name)

    def get(self, name: str) -> torch.Tensor:
        return self._mem[name] if name in self._mem else self._where[name].get(name)


def open_model_dir(model_dir: str) -> Checkpoint:
    paths = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not paths:
        raise SafetensorsError(f"no .safetensors files in {model_dir}")
    return Checkpoint([SafetensorsFile(p) for p in paths])


def save_file(tensors: dict, path: str, metadata: dict | None = None) -> None:
    """Writes CPU tensors under their names, in name order."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    blobs = []
    for name in order:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TAG_OF:
            raise SafetensorsError(f"{name}: element type {t.dtype} cannot be stored")
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _TAG_OF[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
