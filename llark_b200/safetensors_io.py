"""Reader / writer of the safetensors container: 8 bytes little-endian header length, that many bytes of JSON
(name -> {"dtype", "shape", "data_offsets"}, optional "__metadata__"), then the raw little-endian data. Host code; the
file is memory-mapped and every tensor is a view of the map until it is copied to the device."""
import json
import mmap
import struct

import torch

_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
           "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
           "BOOL": torch.bool}
_NAMES = {v: k for k, v in _DTYPES.items()}


def load_file(path):
    """name -> CPU tensor (views of one read-only map of the file; clone or move before the map is dropped)."""
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
    if len(mm) < 8:
        raise ValueError(f"{path}: not a safetensors file")
    (n,) = struct.unpack("<Q", mm[:8])
    if 8 + n > len(mm):
        raise ValueError(f"{path}: header length {n} exceeds the file")
    header = json.loads(bytes(mm[8:8 + n]).decode("utf-8"))
    base = 8 + n
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dtype = _DTYPES.get(meta["dtype"])
        if dtype is None:
            raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
        lo, hi = meta["data_offsets"]
        shape = [int(s) for s in meta["shape"]]
        count = 1
        for s in shape:
            count *= s
        if hi - lo != count * torch.empty((), dtype=dtype).element_size() or base + hi > len(mm):
            raise ValueError(f"{path}: tensor {name!r} does not fit its data_offsets")
        if count == 0:
            out[name] = torch.empty(shape, dtype=dtype)
        else:
            out[name] = torch.frombuffer(mm, dtype=dtype, count=count, offset=base + lo).reshape(shape)
    return out


def save_file(tensors, path, metadata=None):
    header, blobs, at = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""  # a single number has no axis to view
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    js = json.dumps(header, separators=(",", ":")).encode("utf-8")
    js += b" " * ((8 - len(js) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        for raw in blobs:
            f.write(raw)
