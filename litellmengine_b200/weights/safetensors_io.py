"""Reading and writing the safetensors container without any library.

Layout of a file: 8 bytes little-endian header length N; N bytes of JSON
`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}`;
then the raw little-endian tensor bytes, offsets relative to the end of the header.

The reference does not read safetensors itself: a script converts them to one raw
file per tensor plus an index (scripts/convert_weights.py:68-93,143-190) that
src/weights/weight_loader.cpp:122-178 reads; every float type is widened to fp32
there.  Here the container is read in place through a memory map and tensors keep
the type they were stored in until a part binds them.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped .safetensors file: names, shapes, and zero-copy tensors."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from None
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a safetensors header")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + n
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        data_len = size - self._data_start
        for name, e in header.items():
            try:
                dt, shape, (b, en) = e["dtype"], tuple(int(x) for x in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor {name!r}") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            if any(s < 0 for s in shape):
                raise SafetensorsError(f"{path}: tensor {name!r} has a negative dimension {shape}")
            numel = 1
            for s in shape:
                numel *= s
            want = numel * torch.empty((), dtype=_DTYPES[dt]).element_size()
            if not (0 <= b <= en <= data_len) or en - b != want:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} {dt}{list(shape)} needs {want} bytes, "
                    f"data_offsets give [{b}, {en}) of {data_len}")
            self._entries[name] = (_DTYPES[dt], shape, b, en)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self._entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self._entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only; copy before writing)."""
        dt, shape, b, en = self._entries[name]
        if en == b:
            return torch.empty(shape, dtype=dt)
        buf = memoryview(self._mm)[self._data_start + b: self._data_start + en]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")   # torch warns that the buffer is read-only
            t = torch.frombuffer(buf, dtype=dt)
        return t.view(shape)

    def close(self) -> None:
        # Tensors handed out keep the map alive through their memoryview.
        try:
            self._f.close()
        except Exception:
            pass


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write `tensors` (CPU or GPU; made contiguous) to `path` in sorted-name order."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """All safetensors files of a model folder: the shards named by
    `model.safetensors.index.json` if it is there, else every `*.safetensors`."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            try:
                wm = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise SafetensorsError(f"{index}: no weight_map") from None
        files = sorted(set(wm.values()))
    else:
        try:
            files = sorted(fn for fn in os.listdir(model_dir) if fn.endswith(".safetensors"))
        except OSError as e:
            raise SafetensorsError(f"{model_dir}: cannot list ({e.strerror})") from None
    if not files:
        raise SafetensorsError(f"{model_dir}: no .safetensors file")
    return [SafetensorsFile(os.path.join(model_dir, fn)) for fn in files]
