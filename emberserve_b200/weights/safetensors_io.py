"""Reading and writing safetensors files without a helper package.

The format: 8 bytes little-endian header length, a JSON header mapping each tensor name
to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of
the header), then the raw little-endian data.  The reader maps the file and hands out
tensors that view the mapping, so loading a checkpoint copies each tensor once, to the
device.  (The reference goes through the ``safetensors`` package,
``emberserve/model/weights.py:189-199``; ``emberserve/model/fastload.py:12-14``
describes the same layout.)
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from pathlib import Path

import torch

_DTYPES: dict[str, torch.dtype] = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int  # absolute byte offset in the file
    end: int
    file: str


class SafetensorsFile:
    """One mapped ``.safetensors`` file."""

    def __init__(self, path: str | os.PathLike) -> None:
        self.path = str(path)
        size = os.path.getsize(self.path)
        with open(self.path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise SafetensorsError(f"{self.path}: truncated (no header length)")
            (hlen,) = struct.unpack("<Q", head)
            if hlen <= 0 or 8 + hlen > size:
                raise SafetensorsError(f"{self.path}: header length {hlen} exceeds the file")
            try:
                header = json.loads(f.read(hlen))
            except ValueError as e:
                raise SafetensorsError(f"{self.path}: header is not JSON: {e}") from None
            self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        base = 8 + hlen
        self.metadata = header.pop("__metadata__", {}) or {}
        self.tensors: dict[str, TensorInfo] = {}
        for name, meta in header.items():
            if meta["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
            dtype = _DTYPES[meta["dtype"]]
            shape = tuple(int(s) for s in meta["shape"])
            begin, end = (int(o) for o in meta["data_offsets"])
            numel = 1
            for s in shape:
                numel *= s
            esize = torch.empty((), dtype=dtype).element_size()
            if end - begin != numel * esize or base + end > size or begin < 0:
                raise SafetensorsError(
                    f"{self.path}: tensor {name!r} spans bytes [{begin}, {end}) but shape "
                    f"{shape} of {meta['dtype']} needs {numel * esize} (file data is {size - base} bytes)")
            self.tensors[name] = TensorInfo(name, dtype, shape, base + begin, base + end, self.path)

    def names(self) -> list[str]:
        return list(self.tensors)

    def get(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapping (read-only; copy before writing)."""
        info = self.tensors[name]
        numel = 1
        for s in info.shape:
            numel *= s
        if numel == 0:
            return torch.empty(info.shape, dtype=info.dtype)
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only by design
            flat = torch.frombuffer(self._map, dtype=info.dtype, count=numel, offset=info.begin)
        return flat.view(info.shape)

    def close(self) -> None:
        # Tensors handed out keep the mapping alive through the buffer protocol.
        self._map = None


def write_safetensors(path: str | os.PathLike, tensors: dict[str, torch.Tensor],
                      metadata: dict[str, str] | None = None) -> None:
    """Write `tensors` (CPU or device; stored as they are typed) to one file."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs: list[bytes] = []
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} (tensor {name!r})")
        c = t.detach().to("cpu").contiguous()
        raw = c.reshape(-1).view(torch.uint8).numpy().tobytes() if c.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(c.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode()
    hjson += b" " * ((8 - len(hjson) % 8) % 8)  # keep the data 8-byte aligned
    tmp = Path(str(path) + ".tmp")
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)


def open_model_files(model_dir: str | os.PathLike) -> list[SafetensorsFile]:
    """Every ``*.safetensors`` of the folder, sorted by name."""
    paths = sorted(Path(model_dir).glob("*.safetensors"))
    if not paths:
        raise FileNotFoundError(f"no *.safetensors files in {model_dir}")
    return [SafetensorsFile(p) for p in paths]
