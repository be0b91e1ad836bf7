"""Reading and writing the safetensors container, by tensor name.

Layout: 8 bytes little-endian header length N, N bytes of JSON
{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}, then the
data, offsets relative to its start.  A folder may hold one ``model.safetensors`` or
shards named by ``model.safetensors.index.json`` ("weight_map": name -> file).
The reference leaves this to ``from_pretrained``
(src/flexengine/inference/models/qwen2.py:51-65); here it is read directly so that
missing, unexpected and misshapen tensors can be reported by name.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass

import torch

DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
          "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
          "BOOL": torch.bool}
NAMES = {v: k for k, v in DTYPES.items()}


class CheckpointFormatError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: tuple
    file: str
    begin: int      # absolute byte offset in the file
    nbytes: int


class CheckpointReader:
    """Index of every tensor in a model folder; tensors are read on demand from a mapping."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.entries: dict[str, TensorEntry] = {}
        self._maps: dict[str, mmap.mmap] = {}
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        if os.path.isfile(index):
            with open(index, "r", encoding="utf8") as f:
                files = sorted(set(json.load(f).get("weight_map", {}).values()))
        elif os.path.isfile(single):
            files = ["model.safetensors"]
        else:
            files = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors")) \
                if os.path.isdir(model_dir) else []
        if not files:
            raise CheckpointFormatError(f"no model.safetensors (or shard index) in {model_dir!r}")
        for name in files:
            self._index_file(os.path.join(model_dir, name))

    def _index_file(self, path: str) -> None:
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise CheckpointFormatError(f"{path}: too short for a safetensors header")
            (n,) = struct.unpack("<Q", head)
            if n <= 0 or 8 + n > size:
                raise CheckpointFormatError(f"{path}: header length {n} does not fit the file")
            try:
                header = json.loads(f.read(n).decode("utf8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as ex:
                raise CheckpointFormatError(f"{path}: header is not JSON: {ex}") from ex
        base = 8 + n
        for name, info in header.items():
            if name == "__metadata__":
                continue
            begin, end = info["data_offsets"]
            dtype = info["dtype"]
            if dtype not in DTYPES:
                raise CheckpointFormatError(f"{path}: tensor {name!r} has unsupported dtype {dtype}")
            shape = tuple(int(s) for s in info["shape"])
            count = 1
            for s in shape:
                count *= s
            want = count * torch.empty((), dtype=DTYPES[dtype]).element_size()
            if end - begin != want or base + end > size:
                raise CheckpointFormatError(f"{path}: tensor {name!r} data range does not match its shape")
            if name in self.entries:
                raise CheckpointFormatError(f"tensor {name!r} appears in more than one file")
            self.entries[name] = TensorEntry(name, dtype, shape, path, base + begin, end - begin)

    def names(self):
        return self.entries.keys()

    def read(self, name: str) -> torch.Tensor:
        """The tensor as a CPU tensor backed by a private mapping of the file (not a copy)."""
        e = self.entries[name]
        if e.file not in self._maps:
            with open(e.file, "rb") as f:
                self._maps[e.file] = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
        if e.nbytes == 0:
            return torch.empty(e.shape, dtype=DTYPES[e.dtype])
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            flat = torch.frombuffer(self._maps[e.file], dtype=DTYPES[e.dtype],
                                    count=e.nbytes // torch.empty((), dtype=DTYPES[e.dtype]).element_size(),
                                    offset=e.begin)
        return flat.view(e.shape)

    def close(self) -> None:
        self._maps.clear()


def write_safetensors(path: str, named_shapes: list, produce, metadata: dict | None = None) -> None:
    """Write tensors one after another without holding them all.

    ``named_shapes``: [(name, shape, torch dtype)] in file order; ``produce(name)`` returns the
    tensor (CPU, that shape and dtype) when its turn comes.
    """
    header, offset = {}, 0
    for name, shape, dtype in named_shapes:
        count = 1
        for s in shape:
            count *= int(s)
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        header[name] = {"dtype": NAMES[dtype], "shape": [int(s) for s in shape],
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf8")
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, shape, dtype in named_shapes:
            t = produce(name)
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise ValueError(f"produce({name!r}) returned {tuple(t.shape)} {t.dtype}, want {tuple(shape)} {dtype}")
            t = t.contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
