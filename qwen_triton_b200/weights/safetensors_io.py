"""Reading and writing safetensors model folders by tensor name.

File discovery follows the reference loader (qwen_triton/loaders/hf.py:59-70):
``model.safetensors.index.json`` names the shard files, else every
``*.safetensors`` file of the folder is read.  Only headers are parsed up
front; tensor data is read one tensor at a time.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from pathlib import Path

import torch

_DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_DTYPE_NAMES = {v: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class StoredTensor:
    file: Path
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int   # absolute byte offsets in the file
    end: int


def _read_header(path: Path) -> dict[str, StoredTensor]:
    with path.open("rb") as handle:
        (header_len,) = struct.unpack("<Q", handle.read(8))
        header = json.loads(handle.read(header_len).decode("utf-8"))
    base = 8 + header_len
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if meta["dtype"] not in _DTYPES:
            raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
        begin, end = meta["data_offsets"]
        out[name] = StoredTensor(path, _DTYPES[meta["dtype"]], tuple(meta["shape"]), base + begin, base + end)
    return out


def checkpoint_files(folder: Path) -> list[Path]:
    folder = Path(folder)
    index = folder / "model.safetensors.index.json"
    if index.exists():
        with index.open("r", encoding="utf-8") as handle:
            weight_map = json.load(handle)["weight_map"]
        return sorted({folder / name for name in weight_map.values()})
    files = sorted(folder.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files found under {folder}")
    return files


class Checkpoint:
    """Index of every tensor stored in a model folder; reads single tensors on demand."""

    def __init__(self, folder: str | Path) -> None:
        self.folder = Path(folder)
        self.tensors: dict[str, StoredTensor] = {}
        for path in checkpoint_files(self.folder):
            for name, stored in _read_header(path).items():
                if name in self.tensors:
                    raise ValueError(f"tensor {name!r} is stored twice ({self.tensors[name].file} and {path})")
                self.tensors[name] = stored

    def names(self) -> list[str]:
        return sorted(self.tensors)

    def read(self, name: str) -> torch.Tensor:
        stored = self.tensors[name]
        count = 1
        for dim in stored.shape:
            count *= dim
        with stored.file.open("rb") as handle:
            handle.seek(stored.begin)
            data = bytearray(handle.read(stored.end - stored.begin))
        if count == 0:
            return torch.empty(stored.shape, dtype=stored.dtype)
        return torch.frombuffer(data, dtype=stored.dtype, count=count).reshape(stored.shape)


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor]) -> None:
    """Write ``tensors`` (any listed dtype) as one safetensors file, names sorted."""
    write_safetensors_from(path, {name: (t.dtype, tuple(t.shape)) for name, t in tensors.items()}, tensors.__getitem__)


def write_safetensors_from(path: str | Path, entries: dict[str, tuple[torch.dtype, tuple[int, ...]]], produce) -> None:
    """The same file from ``produce(name) -> tensor``, called once per tensor in the order they are written, so
    that a model larger than the host would like to hold at once can be written tensor by tensor."""
    header: dict[str, dict] = {}
    offset = 0
    order = sorted(entries)
    for name in order:
        dtype, shape = entries[name]
        if dtype not in _DTYPE_NAMES:
            raise ValueError(f"cannot store dtype {dtype}")
        count = 1
        for dim in shape:
            count *= dim
        size = count * torch.empty((), dtype=dtype).element_size()
        header[name] = {"dtype": _DTYPE_NAMES[dtype], "shape": list(shape), "data_offsets": [offset, offset + size]}
        offset += size
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with Path(path).open("wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for name in order:
            dtype, shape = entries[name]
            tensor = produce(name).detach().contiguous().cpu()
            if tensor.dtype != dtype or tuple(tensor.shape) != tuple(shape):
                raise ValueError(f"{name}: produced {tensor.dtype} {tuple(tensor.shape)}, declared {dtype} {tuple(shape)}")
            if tensor.numel():
                handle.write(memoryview(tensor.reshape(-1).view(torch.uint8).numpy()))
