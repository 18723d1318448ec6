"""Reading and writing safetensors files without any helper package.

File layout: an 8-byte little-endian header length, a JSON header that maps
each tensor name to ``{"dtype", "shape", "data_offsets": [lo, hi]}`` (offsets
relative to the end of the header), then the raw little-endian data.  The
checks follow the reference's folder reader
(crates/esp/src/infer/decoder/checkpoint.rs:22, :47-158): bounded header,
known dtypes, byte count = shape x element size, offsets inside the file,
contiguous and not overlapping.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

from ..errors import InvalidWeights

MAX_HEADER_BYTES = 16 << 20

# safetensors dtype -> (numpy carrier dtype, torch dtype, element bytes)
_DTYPES = {
    "F32": (np.float32, torch.float32, 4),
    "BF16": (np.uint16, torch.bfloat16, 2),
    "F16": (np.float16, torch.float16, 2),
    "I32": (np.int32, torch.int32, 4),
    "I64": (np.int64, torch.int64, 8),
}
_TORCH_TO_ST = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.int32: "I32",
                torch.int64: "I64"}


@dataclass(frozen=True)
class TensorMeta:
    name: str
    dtype: torch.dtype
    shape: tuple
    file: Path
    lo: int          # absolute byte offsets in ``file``
    hi: int


def read_header(path: Path) -> dict:
    """name -> TensorMeta for one file; raises InvalidWeights on a malformed file."""
    path = Path(path)
    size = path.stat().st_size
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise InvalidWeights(f"{path.name}: shorter than a safetensors header")
        (hlen,) = struct.unpack("<Q", head)
        if hlen > MAX_HEADER_BYTES or 8 + hlen > size:
            raise InvalidWeights(f"{path.name}: header length {hlen} is out of bounds")
        try:
            header = json.loads(f.read(hlen))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise InvalidWeights(f"{path.name}: header is not JSON ({e})") from None
    if not isinstance(header, dict):
        raise InvalidWeights(f"{path.name}: header is not a JSON object")
    base = 8 + hlen
    metas, spans = {}, []
    for name, m in header.items():
        if name == "__metadata__":
            continue
        try:
            st, shape, (lo, hi) = m["dtype"], tuple(int(s) for s in m["shape"]), m["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise InvalidWeights(f"{path.name}: malformed entry for {name}") from None
        if st not in _DTYPES:
            raise InvalidWeights(f"{path.name}: {name} has dtype {st}; supported: {sorted(_DTYPES)}")
        count = 1
        for s in shape:
            count *= s
        if any(s < 0 for s in shape) or hi - lo != count * _DTYPES[st][2] or lo < 0 or base + hi > size:
            raise InvalidWeights(f"{path.name}: {name} offsets [{lo}, {hi}) do not match shape {list(shape)} {st}")
        metas[name] = TensorMeta(name, _DTYPES[st][1], shape, path, base + lo, base + hi)
        spans.append((lo, hi, name))
    spans.sort()
    end = 0
    for lo, hi, name in spans:
        if lo != end:
            raise InvalidWeights(f"{path.name}: data of {name} starts at {lo}, expected {end} (gap or overlap)")
        end = hi
    return metas


def open_model_folder(folder) -> dict:
    """name -> TensorMeta over ``model.safetensors`` or, if present, the shards
    listed by ``model.safetensors.index.json`` (whose weight_map must agree
    with the shards' own headers; shard names are plain file names)."""
    folder = Path(folder)
    index = folder / "model.safetensors.index.json"
    single = folder / "model.safetensors"
    if index.is_file():
        try:
            wmap = json.loads(index.read_text())["weight_map"]
        except (json.JSONDecodeError, KeyError, TypeError):
            raise InvalidWeights("model.safetensors.index.json has no weight_map") from None
        metas = {}
        for shard in sorted(set(wmap.values())):
            if "/" in shard or "\\" in shard or shard in ("", ".", ".."):
                raise InvalidWeights(f"shard name {shard!r} is not a plain file name")
            if not (folder / shard).is_file():
                raise InvalidWeights(f"shard {shard} named by the index is missing")
            for name, m in read_header(folder / shard).items():
                if wmap.get(name) != shard:
                    raise InvalidWeights(f"{name} is in {shard} but the index maps it to {wmap.get(name)}")
                metas[name] = m
        lost = sorted(set(wmap) - set(metas))
        if lost:
            raise InvalidWeights(f"the index names tensors that no shard holds: {lost[:8]}")
        return metas
    if single.is_file():
        return read_header(single)
    raise InvalidWeights(f"no model.safetensors (or index) in {folder}")


def read_tensor(meta: TensorMeta) -> torch.Tensor:
    """The tensor's data as a CPU torch tensor of its stored dtype."""
    st = _TORCH_TO_ST[meta.dtype]
    np_dtype = _DTYPES[st][0]
    count = (meta.hi - meta.lo) // _DTYPES[st][2]
    if count == 0:
        return torch.empty(meta.shape, dtype=meta.dtype)
    arr = np.fromfile(meta.file, dtype=np_dtype, count=count, offset=meta.lo)
    t = torch.from_numpy(arr)
    if meta.dtype == torch.bfloat16:
        t = t.view(torch.bfloat16)
    return t.reshape(meta.shape)


def write_safetensors(path, tensors: dict) -> None:
    """``tensors``: name -> CPU torch tensor (float32, bfloat16, float16, int32, int64)."""
    header, offset, blobs = {}, 0, []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_ST:
            raise InvalidWeights(f"{name}: dtype {t.dtype} cannot be written")
        raw = t.view(torch.uint16).numpy().tobytes() if t.dtype == torch.bfloat16 else t.numpy().tobytes()
        header[name] = {"dtype": _TORCH_TO_ST[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    head = json.dumps(header, separators=(",", ":")).encode()
    head += b" " * ((8 - len(head) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for raw in blobs:
            f.write(raw)
