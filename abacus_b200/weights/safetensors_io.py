"""Reading and writing safetensors files, by tensor name.

The container is the one tools/export.py:28-38 parses: an 8-byte little-endian
header length, a JSON header {name: {dtype, shape, data_offsets}}, then the
data, offsets counted from the end of the header. Every *.safetensors file of
a folder is read and the names merged.

Tensors keep the precision they are stored in: BF16 stays bfloat16, F32 stays
float32, integer tables (I32, I64) become int32.
"""
import glob
import json
import mmap
import os
import struct

import torch


class WeightError(ValueError):
    """A weights file that cannot be read, or does not hold what the model needs."""


_DTYPES = {"BF16": (torch.bfloat16, 2), "F32": (torch.float32, 4), "I32": (torch.int32, 4), "I64": (torch.int64, 8)}
_NAMES = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32", torch.int64: "I64"}


def read_header(path):
    """-> (entries {name: (dtype string, shape, begin, end)}, offset of the data, file size)."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise WeightError(f"{path}: truncated (no header length)")
        (n,) = struct.unpack("<Q", head)
        if n > size - 8:
            raise WeightError(f"{path}: header length {n} runs past the end of the file ({size} bytes)")
        try:
            header = json.loads(f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise WeightError(f"{path}: header is not valid JSON ({e})") from None
    entries = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape, (a, b) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise WeightError(f"{path}: malformed header entry for {name!r}") from None
        if dtype not in _DTYPES:
            raise WeightError(f"{path}: tensor {name!r} has dtype {dtype}; only {', '.join(_DTYPES)} are read")
        count = 1
        for s in shape:
            count *= s
        if b - a != count * _DTYPES[dtype][1]:
            raise WeightError(f"{path}: tensor {name!r}: {b - a} bytes for shape {list(shape)} of {dtype}")
        if 8 + n + b > size:
            raise WeightError(f"{path}: truncated: tensor {name!r} ends at byte {8 + n + b}, file has {size}")
        entries[name] = (dtype, shape, a, b)
    return entries, 8 + n, size


def folder_files(folder):
    files = sorted(glob.glob(os.path.join(folder, "*.safetensors")))  # tools/export.py:30
    if not files:
        raise WeightError(f"{folder}: no *.safetensors file")
    return files


def folder_index(folder):
    """{name: (path, dtype string, shape, absolute begin, absolute end)} over all files of a folder."""
    index = {}
    for path in folder_files(folder):
        entries, base, _ = read_header(path)
        for name, (dtype, shape, a, b) in entries.items():
            if name in index:
                raise WeightError(f"tensor {name!r} is in both {index[name][0]} and {path}")
            index[name] = (path, dtype, shape, base + a, base + b)
    return index


class FolderReader:
    """Hands out tensors of a folder by name; the files are mapped, not read whole."""

    def __init__(self, folder):
        self.index = folder_index(folder)
        self._maps = {}

    def names(self):
        return list(self.index)

    def shape(self, name):
        return self.index[name][2]

    def dtype(self, name):
        return _DTYPES[self.index[name][1]][0]

    def tensor(self, name):
        path, dtype, shape, a, b = self.index[name]
        if path not in self._maps:
            with open(path, "rb") as f:
                self._maps[path] = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
        tdtype = _DTYPES[dtype][0]
        if b == a:
            t = torch.empty(shape, dtype=tdtype)
        else:
            t = torch.frombuffer(self._maps[path], dtype=tdtype, count=(b - a) // _DTYPES[dtype][1], offset=a).reshape(shape)
        return t.to(torch.int32) if tdtype == torch.int64 else t


def save_tensors(path, tensors):
    """Write {name: CPU tensor} as one safetensors file."""
    header, offset, blobs = {}, 0, []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightError(f"tensor {name!r}: dtype {t.dtype} cannot be written")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
