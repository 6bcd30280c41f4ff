"""A minimal GGUF v2/v3 writer for the container tests: exactly the bytes the
format description prescribes, with hooks to produce malformed files."""
import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q",
        F64: "<d"}


def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def _payload(vtype: int, v) -> bytes:
    if vtype == STR:
        return _s(v)
    return struct.pack(_FMT[vtype], v)


def kv(key: str, vtype: int, v, elem_type: int | None = None) -> bytes:
    out = _s(key) + struct.pack("<I", vtype)
    if vtype == ARR:
        out += struct.pack("<IQ", elem_type, len(v)) + b"".join(_payload(elem_type, e) for e in v)
    else:
        out += _payload(vtype, v)
    return out


def build(tensors, metadata=(), version=3, alignment=None, magic=b"GGUF", offsets=None, counts=None, pad_to=None) -> bytes:
    """tensors: [(name, dims innermost-first, ggml_type, payload bytes)].  `offsets` overrides the
    per-tensor data offsets, `counts` the (tensor, kv) counts written in the header."""
    align = 32 if not alignment else alignment  # the file's layout; the key is written as given
    kvs = list(metadata)
    if alignment is not None:
        kvs.append(kv("general.alignment", U32, alignment))
    n_t, n_kv = counts if counts else (len(tensors), len(kvs))
    head = magic + struct.pack("<IQQ", version, n_t, n_kv) + b"".join(kvs)
    offs, cur = [], 0
    for _, _, _, data in tensors:
        offs.append(cur)
        cur = (cur + len(data) + align - 1) // align * align
    if offsets is not None:
        offs = list(offsets)
    for (name, dims, ty, _), off in zip(tensors, offs):
        head += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", ty, off)
    start = (len(head) + align - 1) // align * align
    blob = bytearray(head + b"\0" * (start - len(head)))
    for (_, _, _, data), off in zip(tensors, offs):
        end = start + off + len(data)
        if off > (1 << 28):  # a lying offset: the payload is simply not in the file
            continue
        if len(blob) < end:
            blob += b"\0" * (end - len(blob))
        blob[start + off:end] = data
    if pad_to is not None:
        blob = blob[:pad_to] if pad_to < len(blob) else blob + b"\0" * (pad_to - len(blob))
    return bytes(blob)


def as_bytes(a) -> bytes:
    return np.ascontiguousarray(a).tobytes()
