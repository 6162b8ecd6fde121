"""Reading and writing the safetensors container, by tensor name.

The format: an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` (plus an optional
``__metadata__`` entry), then the raw little-endian tensor bytes.  A model
folder holds one ``model.safetensors`` or several shards named by
``model.safetensors.index.json`` (``weight_map``: tensor name -> file).

davidjoyme/flashdecode-cuda reaches its weights through
``AutoModelForCausalLM.from_pretrained(...).state_dict()`` (engine/loader.py:20-27);
this reader needs neither that package nor a network.
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


def read_header(path: Path) -> Tuple[Dict[str, dict], int]:
    """(header without ``__metadata__``, offset of the data section)."""
    size = path.stat().st_size
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: shorter than a safetensors header")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header is not a JSON object")
    header.pop("__metadata__", None)
    data_len = size - 8 - n
    for name, info in header.items():
        try:
            dt, shape, (b, e) = info["dtype"], info["shape"], info["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: entry {name!r} lacks dtype/shape/data_offsets") from None
        if dt not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt}")
        count = 1
        for s in shape:
            count *= int(s)
        want = count * torch.empty((), dtype=_DTYPES[dt]).element_size()
        if not (0 <= b <= e <= data_len) or e - b != want:
            raise SafetensorsError(f"{path}: tensor {name!r} offsets [{b}, {e}) do not match "
                                   f"shape {shape} of {dt} ({want} bytes) within {data_len} bytes of data")
    return header, 8 + n


def read_file(path: Path) -> Dict[str, torch.Tensor]:
    """All tensors of one file, on the CPU, in their stored dtype.  The
    tensors are views of a private (copy-on-write) mapping of the file."""
    path = Path(path)
    header, base = read_header(path)
    out: Dict[str, torch.Tensor] = {}
    if not header:
        return out
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
    for name, info in header.items():
        dtype = _DTYPES[info["dtype"]]
        shape = [int(s) for s in info["shape"]]
        b, e = info["data_offsets"]
        count = 1
        for s in shape:
            count *= s
        if count == 0:
            out[name] = torch.empty(shape, dtype=dtype)
        else:
            out[name] = torch.frombuffer(mm, dtype=dtype, count=count, offset=base + b).view(shape)
    return out


def read_folder(folder: Path) -> Dict[str, torch.Tensor]:
    """All tensors of a model folder: ``model.safetensors`` or the shards an
    index names."""
    folder = Path(folder)
    index = folder / "model.safetensors.index.json"
    single = folder / "model.safetensors"
    if index.exists():
        weight_map = json.loads(index.read_text()).get("weight_map", {})
        out: Dict[str, torch.Tensor] = {}
        for shard in sorted(set(weight_map.values())):
            tensors = read_file(folder / shard)
            for name, t in tensors.items():
                if weight_map.get(name) == shard:
                    out[name] = t
        lost = sorted(set(weight_map) - set(out))
        if lost:
            raise SafetensorsError(f"{index}: tensors named by the index but found in no shard: {lost[:8]}")
        return out
    if single.exists():
        return read_file(single)
    raise FileNotFoundError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")


def write_file(path: Path, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write tensors (any device) in name order."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))


def names_of(tensors: Iterable[str]) -> list:
    return sorted(tensors)
