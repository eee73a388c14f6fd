"""Reading and writing the safetensors container.

Layout: 8 bytes little-endian header length, a JSON header
`{name: {dtype, shape, data_offsets:[begin, end]}, "__metadata__": {...}}`, then
the data.  A folder holds one `model.safetensors` or several shards listed in
`model.safetensors.index.json` under `weight_map` (src/safetensors.rs:65-103).
Every offset is checked against the file before anything is read
(src/safetensors.rs:119-150).  Files are memory-mapped; a tensor is a view of
the mapping until it is copied to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

from ..errors import FormatError, IoError, MissingTensorError

# container dtype tag -> (torch dtype, bytes per element)
DTYPES: Dict[str, Tuple[torch.dtype, int]] = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_TAG_OF = {v[0]: k for k, v in DTYPES.items()}

SINGLE_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"


@dataclass(frozen=True)
class TensorEntry:
    shard: int
    dtype: str
    shape: Tuple[int, ...]
    begin: int     # absolute byte offsets into the shard
    end: int


class SafetensorsFolder:
    """All tensors of a model folder, by name."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self._maps: List[mmap.mmap] = []
        self._files = []
        self.entries: Dict[str, TensorEntry] = {}
        index_path = os.path.join(model_dir, INDEX_FILE)
        if os.path.exists(index_path):
            idx = _read_json(index_path)
            wm = idx.get("weight_map") if isinstance(idx, dict) else None
            if not isinstance(wm, dict):
                raise FormatError(f"malformed file: {index_path} has no weight_map")
            shards = sorted({v for v in wm.values() if isinstance(v, str)})
            if not shards:
                raise FormatError(f"malformed file: {index_path} lists no shard")
            for fname in shards:
                self._add_shard(os.path.join(model_dir, fname))
        else:
            single = os.path.join(model_dir, SINGLE_FILE)
            if not os.path.exists(single):
                raise FormatError(f"malformed file: no safetensors in {model_dir} "
                                  f"(need {SINGLE_FILE} or {INDEX_FILE})")
            self._add_shard(single)

    def _add_shard(self, path: str) -> None:
        try:
            f = open(path, "rb")
            size = os.fstat(f.fileno()).st_size
        except OSError as e:
            raise IoError(f"io error: {path}: {e.strerror or e}") from e
        if size < 8:
            f.close()
            raise FormatError(f"malformed file: {path} too small")
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        hlen = struct.unpack("<Q", mm[:8])[0]
        data_base = 8 + hlen
        if data_base > size:
            raise FormatError(f"malformed file: {path}: header out of bounds")
        try:
            header = json.loads(bytes(mm[8:data_base]))
        except ValueError as e:
            raise FormatError(f"malformed file: {path}: bad header json: {e}") from e
        if not isinstance(header, dict):
            raise FormatError(f"malformed file: {path}: header is not an object")
        shard = len(self._maps)
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            if not isinstance(meta, dict):
                raise FormatError(f"malformed file: {path}: {name}: entry is not an object")
            tag = meta.get("dtype")
            if tag not in DTYPES:
                raise FormatError(f"malformed file: {path}: {name}: dtype {tag!r} unsupported "
                                  f"({'/'.join(DTYPES)} only)")
            shape = meta.get("shape")
            if not isinstance(shape, list) or not all(isinstance(s, int) and s >= 0 for s in shape):
                raise FormatError(f"malformed file: {path}: {name}: no shape")
            off = meta.get("data_offsets")
            if (not isinstance(off, list) or len(off) != 2
                    or not all(isinstance(o, int) and o >= 0 for o in off)):
                raise FormatError(f"malformed file: {path}: {name}: no data_offsets")
            begin, end = data_base + off[0], data_base + off[1]
            if begin > end or end > size:
                raise FormatError(f"malformed file: {path}: {name}: data out of bounds")
            numel = 1
            for s in shape:
                numel *= s
            if numel * DTYPES[tag][1] != end - begin:
                raise FormatError(f"malformed file: {path}: {name}: {end - begin} bytes do not hold "
                                  f"shape {shape} of {tag}")
            if name in self.entries:
                raise FormatError(f"malformed file: {path}: {name}: tensor appears in two shards")
            self.entries[name] = TensorEntry(shard, tag, tuple(shape), begin, end)
        self._maps.append(mm)
        self._files.append(f)

    # -- the tensor-source interface --------------------------------------------------
    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        e = self.entries.get(name)
        if e is None:
            raise MissingTensorError(f"missing tensor '{name}'")
        return DTYPES[e.dtype][0], e.shape

    def read(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapping (read-only memory: copy before writing)."""
        e = self.entries.get(name)
        if e is None:
            raise MissingTensorError(f"missing tensor '{name}'")
        dtype = DTYPES[e.dtype][0]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=dtype)
        view = memoryview(self._maps[e.shard])[e.begin:e.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # torch warns that the buffer is not writable
            t = torch.frombuffer(view, dtype=dtype)
        return t.view(e.shape)

    def close(self) -> None:
        self.entries.clear()
        for mm in self._maps:
            try:
                mm.close()
            except BufferError:
                pass            # a tensor still views it; the mapping goes with the tensor
        for f in self._files:
            f.close()
        self._maps, self._files = [], []


def _read_json(path: str):
    try:
        with open(path, "rb") as f:
            return json.loads(f.read())
    except OSError as e:
        raise IoError(f"io error: {path}: {e.strerror or e}") from e
    except ValueError as e:
        raise FormatError(f"malformed file: {path}: {e}") from e


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Mapping[str, str] = None) -> None:
    """Write tensors (any iterable of (name, CPU tensor), consumed once, so that a
    large model is never held whole) to one file.  Data begins 8-byte aligned."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    tmp_data = path + ".data.tmp"
    offset = 0
    with open(tmp_data, "wb") as d:
        for name, t in tensors:
            if t.dtype not in _TAG_OF:
                raise FormatError(f"cannot store {name}: dtype {t.dtype} unsupported")
            t = t.detach().contiguous().cpu()
            raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
            header[name] = {"dtype": _TAG_OF[t.dtype], "shape": list(t.shape),
                            "data_offsets": [offset, offset + len(raw)]}
            d.write(raw)
            offset += len(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode()
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(path, "wb") as out, open(tmp_data, "rb") as d:
        out.write(struct.pack("<Q", len(hjson)))
        out.write(hjson)
        while True:
            chunk = d.read(1 << 24)
            if not chunk:
                break
            out.write(chunk)
    os.remove(tmp_data)
