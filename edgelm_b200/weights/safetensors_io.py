"""Reading and writing safetensors files, by tensor name, without a dependency.

Format (as adarsh-sgh/edgelm's exporter reads it, tools/export.py:18-41): an unsigned 64-bit
little-endian header length, a JSON header {name: {dtype, shape, data_offsets}}, then the raw
little-endian tensor bytes, offsets counted from the end of the header.
"""
import json
import mmap
import os
import struct
import warnings

import torch

from .errors import WeightsError

_DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


def read_file(path):
    """name -> CPU tensor in the stored dtype (a view of the mapped file, read-only by agreement)."""
    size = os.path.getsize(path)
    if size < 8:
        raise WeightsError(f"{path}: too short to be a safetensors file ({size} bytes)")
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        if n <= 0 or 8 + n > size:
            raise WeightsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise WeightsError(f"{path}: the header is not JSON: {e}") from None
        mapped = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    base = 8 + n
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dt = meta.get("dtype")
        if dt not in _DTYPES:
            raise WeightsError(f"{path}: tensor '{name}' has dtype {dt}, which is not read here")
        shape = [int(s) for s in meta["shape"]]
        b, e = meta["data_offsets"]
        dtype = _DTYPES[dt]
        count = 1
        for s in shape:
            count *= s
        itemsize = torch.empty(0, dtype=dtype).element_size()
        if e - b != count * itemsize or base + e > size or b < 0:
            raise WeightsError(f"{path}: tensor '{name}' of shape {shape} and dtype {dt} does not match its byte range [{b}, {e})")
        if count == 0:
            out[name] = torch.empty(shape, dtype=dtype)
            continue
        with warnings.catch_warnings():  # the mapping is read-only; nothing here writes to it
            warnings.simplefilter("ignore")
            t = torch.frombuffer(mapped, dtype=dtype, count=count, offset=base + b)
        out[name] = t.reshape(shape)
    return out


def read_dir(model_dir):
    """All *.safetensors files of a folder, merged in sorted order (tools/export.py:57-63)."""
    files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if not files:
        raise WeightsError(f"{model_dir}: no .safetensors file")
    out = {}
    for fn in files:
        out.update(read_file(os.path.join(model_dir, fn)))
    return out


def write_file(path, tensors, metadata=None):
    """Write name -> tensor (any device) as one safetensors file, tensors 64-byte aligned."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    plan = []
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise WeightsError(f"tensor '{name}' has dtype {t.dtype}, which is not written here")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        plan.append((name, t, nbytes))
        offset += nbytes
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((-(8 + len(h))) % 64)
    tmp = f"{path}.tmp{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for name, t, nbytes in plan:
            c = t.detach().contiguous().cpu()
            f.write(c.view(torch.uint8).numpy().tobytes() if c.numel() else b"")
    os.replace(tmp, path)
