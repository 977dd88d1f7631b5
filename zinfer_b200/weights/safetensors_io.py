"""Reader and writer of the safetensors container.

Layout: 8-byte little-endian header length, a JSON object mapping tensor names to
``dtype``/``shape``/``data_offsets`` (plus an optional ``__metadata__`` string map),
then the raw data.  The checks are the reference's
(src/format/safetensors.zig:188-234 header, :250-283 entries, :285-327 layout):
every tensor must lie within the data, have exactly ``prod(shape) * itemsize``
bytes, overlap no other, and together they must cover the data without gaps.
The file is memory-mapped, so a tensor's bytes are read when it is copied to the
device and never held twice on the host.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# name -> (bytes per element, numpy dtype used to view the bytes, torch dtype)
_DTYPES = {
    "BF16": (2, np.uint16, torch.bfloat16),
    "F16": (2, np.float16, torch.float16),
    "F32": (4, np.float32, torch.float32),
    "F64": (8, np.float64, torch.float64),
    "I8": (1, np.int8, torch.int8),
    "U8": (1, np.uint8, torch.uint8),
    "I16": (2, np.int16, torch.int16),
    "I32": (4, np.int32, torch.int32),
    "I64": (8, np.int64, torch.int64),
    "BOOL": (1, np.bool_, torch.bool),
}
_NAME_OF = {v[2]: k for k, v in _DTYPES.items()}
MAX_HEADER_BYTES = 100 * 1024 * 1024


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: tuple[int, ...]
    begin: int
    end: int

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][2]


class SafetensorsFile:
    """An open, validated safetensors file; ``tensor(name)`` gives a CPU tensor
    that views the mapping (copy it before the file is closed)."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = self._f.seek(0, 2)
        if size < 8:
            raise SafetensorsError(f"{path}: shorter than the 8-byte header length")
        self._f.seek(0)
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen == 0 or hlen > MAX_HEADER_BYTES:
            raise SafetensorsError(f"{path}: implausible header length {hlen}")
        if 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self.data_start = 8 + hlen
        self.data_size = size - self.data_start
        self.metadata = header.pop("__metadata__", None) or {}
        if not isinstance(self.metadata, dict) or any(not isinstance(v, str) for v in self.metadata.values()):
            raise SafetensorsError(f"{path}: __metadata__ must map strings to strings")
        self.tensors: dict[str, TensorInfo] = {}
        for name, entry in header.items():
            self.tensors[name] = self._parse_entry(name, entry)
        self._validate_layout()
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def _parse_entry(self, name: str, entry) -> TensorInfo:
        p = self.path
        if not isinstance(entry, dict):
            raise SafetensorsError(f"{p}: entry {name!r} is not an object")
        for k in ("dtype", "shape", "data_offsets"):
            if k not in entry:
                raise SafetensorsError(f"{p}: entry {name!r} lacks {k!r}")
        dtype, shape, off = entry["dtype"], entry["shape"], entry["data_offsets"]
        if dtype not in _DTYPES:
            raise SafetensorsError(f"{p}: entry {name!r} has unsupported dtype {dtype!r}")
        if not isinstance(shape, list) or any(not isinstance(s, int) or isinstance(s, bool) or s < 0 for s in shape):
            raise SafetensorsError(f"{p}: entry {name!r} has an invalid shape {shape!r}")
        if (not isinstance(off, list) or len(off) != 2
                or any(not isinstance(o, int) or isinstance(o, bool) or o < 0 for o in off) or off[0] > off[1]):
            raise SafetensorsError(f"{p}: entry {name!r} has invalid data_offsets {off!r}")
        return TensorInfo(name, dtype, tuple(shape), off[0], off[1])

    def _validate_layout(self) -> None:
        p = self.path
        cursor = 0
        for t in sorted(self.tensors.values(), key=lambda t: (t.begin, t.end)):
            if t.end > self.data_size:
                raise SafetensorsError(f"{p}: tensor {t.name!r} ends at {t.end}, beyond the data ({self.data_size} bytes)")
            want = int(np.prod(t.shape, dtype=np.int64)) * _DTYPES[t.dtype][0]
            if t.end - t.begin != want:
                raise SafetensorsError(
                    f"{p}: tensor {t.name!r} of shape {list(t.shape)} {t.dtype} needs {want} bytes, has {t.end - t.begin}")
            if t.begin < cursor:
                raise SafetensorsError(f"{p}: tensor {t.name!r} overlaps the tensor before it")
            if t.begin > cursor:
                raise SafetensorsError(f"{p}: {t.begin - cursor} unused bytes before tensor {t.name!r}")
            cursor = t.end
        if cursor != self.data_size:
            raise SafetensorsError(f"{p}: {self.data_size - cursor} unused bytes after the last tensor")

    def names(self) -> list[str]:
        return list(self.tensors)

    def tensor(self, name: str) -> torch.Tensor:
        t = self.tensors.get(name)
        if t is None:
            raise KeyError(f"{self.path}: no tensor named {name!r}")
        _, npdt, tdt = _DTYPES[t.dtype]
        count = int(np.prod(t.shape, dtype=np.int64))
        if count == 0:
            return torch.empty(t.shape, dtype=tdt)
        arr = np.frombuffer(self._map, dtype=npdt, count=count, offset=self.data_start + t.begin)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; nothing writes through the view
            ten = torch.from_numpy(arr)
        if t.dtype == "BF16":
            ten = ten.view(torch.bfloat16)
        return ten.reshape(t.shape)

    def close(self) -> None:
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:  # views still alive; the mapping goes with them
                pass
            self._map = None
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    """Write tensors in the order given, contiguous and without padding between them."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().to("cpu").contiguous()
        if t.dtype not in _NAME_OF:
            raise SafetensorsError(f"cannot store dtype {t.dtype} ({name!r})")
        raw = t.view(torch.uint16).numpy().tobytes() if t.dtype == torch.bfloat16 else t.numpy().tobytes()
        header[name] = {"dtype": _NAME_OF[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * (-len(hjson) % 8)  # readers trim trailing spaces (safetensors.zig:203-206)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
