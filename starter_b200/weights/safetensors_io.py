"""Reading and writing the safetensors container: an 8-byte little-endian header length, a JSON
header ``{name: {"dtype", "shape", "data_offsets"}}`` and one flat byte buffer.

Tensors are mapped, not read: a tensor's bytes are touched when it is copied to
the device.  Nothing here depends on a model.
"""

from __future__ import annotations

import json
import mmap
import os
import struct

import torch

_DTYPES = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped ``.safetensors`` file; ``entries`` maps a name to (dtype, shape)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        with open(path, "rb") as handle:
            (header_len,) = struct.unpack("<Q", handle.read(8))
            if header_len <= 0 or 8 + header_len > size:
                raise SafetensorsError(f"{path}: header length {header_len} does not fit the file")
            try:
                header = json.loads(handle.read(header_len).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as exc:
                raise SafetensorsError(f"{path}: header is not JSON ({exc})") from None
            self._map = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_COPY)
        self._data_start = 8 + header_len
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries = {}
        self._offsets = {}
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
            dtype = _DTYPES[info["dtype"]]
            shape = tuple(int(d) for d in info["shape"])
            begin, end = (int(v) for v in info["data_offsets"])
            count = 1
            for d in shape:
                count *= d
            if end - begin != count * dtype.itemsize or self._data_start + end > size or begin < 0:
                raise SafetensorsError(f"{path}: tensor {name} has inconsistent offsets")
            self.entries[name] = (dtype, shape)
            self._offsets[name] = (begin, count)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor over the mapped bytes (copy-on-write: writing to it never reaches the file)."""
        dtype, shape = self.entries[name]
        begin, count = self._offsets[name]
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        flat = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._data_start + begin)
        return flat.view(shape)


def write_safetensors(path: str, tensors, metadata: dict | None = None) -> None:
    """Write ``tensors`` (a dict or an iterable of ``(name, cpu tensor)``) in the given order.

    The header is laid out first from shapes and dtypes, so an iterable may produce
    its tensors one at a time and the whole model never has to sit in memory; for
    that, pass ``tensors`` as a ``(layout, producer)`` pair where ``layout`` is a
    list of ``(name, dtype, shape)`` and ``producer(name)`` returns the tensor.
    """
    if isinstance(tensors, tuple) and len(tensors) == 2 and callable(tensors[1]):
        layout, producer = tensors
    else:
        items = dict(tensors)
        layout = [(n, t.dtype, tuple(t.shape)) for n, t in items.items()]
        producer = items.__getitem__
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, dtype, shape in layout:
        if dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name}: dtype {dtype} cannot be stored")
        count = 1
        for d in shape:
            count *= int(d)
        nbytes = count * dtype.itemsize
        header[name] = {
            "dtype": _NAMES[dtype],
            "shape": [int(d) for d in shape],
            "data_offsets": [offset, offset + nbytes],
        }
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for name, dtype, shape in layout:
            tensor = producer(name)
            if tensor.dtype != dtype or tuple(tensor.shape) != tuple(shape):
                raise SafetensorsError(f"tensor {name}: produced {tensor.dtype}{tuple(tensor.shape)}, "
                                       f"announced {dtype}{tuple(shape)}")
            tensor = tensor.detach().contiguous().cpu()
            handle.write(tensor.reshape(-1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)


def open_model_files(model_dir: str) -> dict:
    """Map every tensor name in ``model_dir`` to the ``SafetensorsFile`` that holds it.

    Uses ``model.safetensors.index.json`` when present, else every ``*.safetensors``
    file of the folder.  A name that two files hold is an error.
    """
    index_path = os.path.join(model_dir, "model.safetensors.index.json")
    files = {}
    owners = {}
    if os.path.isfile(index_path):
        with open(index_path, "r", encoding="utf-8") as handle:
            weight_map = json.load(handle)["weight_map"]
        for name, fname in weight_map.items():
            if fname not in files:
                files[fname] = SafetensorsFile(os.path.join(model_dir, fname))
            if name not in files[fname].entries:
                raise SafetensorsError(f"{index_path} places {name} in {fname}, which does not hold it")
            owners[name] = files[fname]
        return owners
    names = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if not names:
        raise SafetensorsError(f"no .safetensors file in {model_dir}")
    for fname in names:
        handle = SafetensorsFile(os.path.join(model_dir, fname))
        for name in handle.entries:
            if name in owners:
                raise SafetensorsError(f"tensor {name} is stored in both {owners[name].path} and {handle.path}")
            owners[name] = handle
    return owners
