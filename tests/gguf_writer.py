"""Minimal GGUF (version 3) writer for the tests: scalar and string metadata, tensors of raw bytes.

Layout (the public GGUF specification): magic "GGUF", version, tensor count, key/value count; key/value pairs
(string key, value type, value); tensor infos (name, n_dims, dims innermost first, ggml type, offset into the data
section); padding to general.alignment; tensor data, each tensor aligned.
"""
import struct

import numpy as np

_T_U32, _T_F32, _T_STR, _T_U64 = 4, 6, 8, 10


def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, meta: dict, tensors: list, alignment: int = 32):
    """meta: key -> int | float | str; tensors: [(name, ggml_type, dims_innermost_first, bytes-like)]."""
    out = bytearray()
    meta = dict(meta)
    meta.setdefault("general.alignment", alignment)
    out += struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(meta))
    for k, v in meta.items():
        out += _s(k.encode())
        if isinstance(v, str):
            out += struct.pack("<I", _T_STR) + _s(v.encode())
        elif isinstance(v, float):
            out += struct.pack("<If", _T_F32, v)
        elif v >= 2 ** 32:
            out += struct.pack("<IQ", _T_U64, v)
        else:
            out += struct.pack("<II", _T_U32, v)
    blobs = [bytes(np.ascontiguousarray(d).view(np.uint8)) if isinstance(d, np.ndarray) else bytes(d) for _, _, _, d in tensors]
    offsets, off = [], 0
    for b in blobs:
        offsets.append(off)
        off = (off + len(b) + alignment - 1) // alignment * alignment
    for (name, ty, dims, _), o in zip(tensors, offsets):
        out += _s(name.encode()) + struct.pack("<I", len(dims))
        for d in dims:
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", ty, o)
    out += b"\0" * ((-len(out)) % alignment)
    for b in blobs:
        out += b
        out += b"\0" * ((-len(b)) % alignment)
    with open(path, "wb") as f:
        f.write(out)
