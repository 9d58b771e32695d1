"""A small reader and writer for the safetensors container.

Layout: 8 bytes little-endian header length ``n``, ``n`` bytes of JSON mapping each tensor
name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of
the header), then the raw little-endian tensor bytes.  The reference reads the same files
through ``safetensors.torch.load_file`` (``clockwork/engine/loader.py:47-54``); this reader
maps the file and hands out tensors one by one so that a model larger than host memory's
free part can still be uploaded tensor by tensor.
"""

from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import torch

_DTYPES: dict[str, torch.dtype] = {
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


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int  # absolute byte offsets in the file
    end: int
    file: Path


class SafetensorsFile:
    """One mapped ``.safetensors`` file."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: truncated (only {size} bytes)")
        self._fh = open(self.path, "rb")
        (header_len,) = struct.unpack("<Q", self._fh.read(8))
        if header_len <= 0 or 8 + header_len > size:
            raise SafetensorsError(
                f"{self.path}: header length {header_len} does not fit a file of {size} bytes"
            )
        try:
            header = json.loads(self._fh.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{self.path}: header is not valid JSON: {exc}") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        base = 8 + header_len
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            dtype = _DTYPES.get(info.get("dtype"))
            if dtype is None:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unknown dtype {info.get('dtype')!r}")
            shape = tuple(int(s) for s in info["shape"])
            begin, end = (int(x) for x in info["data_offsets"])
            numel = 1
            for s in shape:
                numel *= s
            want = numel * torch.empty((), dtype=dtype).element_size()
            if end - begin != want:
                raise SafetensorsError(
                    f"{self.path}: tensor {name!r} of shape {list(shape)} needs {want} bytes, header gives {end - begin}"
                )
            if base + end > size:
                raise SafetensorsError(
                    f"{self.path}: truncated: tensor {name!r} ends at byte {base + end}, file has {size}"
                )
            self.entries[name] = TensorEntry(name, dtype, shape, base + begin, base + end, self.path)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY) if size else None

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (copy before the file is closed)."""
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = memoryview(self._map)[e.begin : e.end]
        return torch.frombuffer(buf, dtype=e.dtype).reshape(e.shape)

    def close(self) -> None:
        # tensors handed out may still view the map; let the garbage collector unmap it
        self._fh.close()


def save_safetensors(path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    """Write tensors (CPU, any of the known dtypes) in name order, data aligned to 8 bytes."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs: list[bytes] = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)))
        fh.write(text)
        for raw in blobs:
            fh.write(raw)


class CheckpointIndex:
    """All ``*.safetensors`` files of a model folder, merged by tensor name
    (sorted file order, later files win, as ``clockwork/engine/loader.py:47-54`` merges them)."""

    def __init__(self, model_dir: str | Path) -> None:
        self.model_dir = Path(model_dir)
        paths = sorted(self.model_dir.glob("*.safetensors"))
        if not paths:
            raise FileNotFoundError(f"no .safetensors files in {self.model_dir}")
        self.files = [SafetensorsFile(p) for p in paths]
        self.entries: dict[str, tuple[SafetensorsFile, TensorEntry]] = {}
        for f in self.files:
            for name, entry in f.entries.items():
                self.entries[name] = (f, entry)

    def names(self) -> list[str]:
        return sorted(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return self.entries[name][1].shape

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name][1].dtype

    def tensor(self, name: str) -> torch.Tensor:
        return self.entries[name][0].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()
