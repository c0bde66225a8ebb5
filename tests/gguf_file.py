"""Writes small GGUF v3 files for the loader tests, from the published layout (the reference has a C++ writer for
its own tests, tests/gguf_writer.h; this is an independent numpy one)."""
import struct

import numpy as np

VT_U32, VT_I32, VT_F32, VT_BOOL, VT_STR, VT_ARR, VT_U64 = 4, 5, 6, 7, 8, 9, 10


def _s(b: str) -> bytes:
    e = b.encode()
    return struct.pack("<Q", len(e)) + e


def write_gguf(path, kvs, tensors, alignment=32, version=3):
    """kvs: list of (key, kind, value) with kind in u32/i32/f32/bool/str/u64/arr_str/arr_i32;
    tensors: list of (name, dims innermost first, ggml type, bytes)."""
    out = bytearray()
    out += struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(kvs))
    for key, kind, v in kvs:
        out += _s(key)
        if kind == "u32": out += struct.pack("<II", VT_U32, v)
        elif kind == "i32": out += struct.pack("<Ii", VT_I32, v)
        elif kind == "f32": out += struct.pack("<If", VT_F32, v)
        elif kind == "bool": out += struct.pack("<IB", VT_BOOL, 1 if v else 0)
        elif kind == "u64": out += struct.pack("<IQ", VT_U64, v)
        elif kind == "str": out += struct.pack("<I", VT_STR) + _s(v)
        elif kind == "arr_str":
            out += struct.pack("<IIQ", VT_ARR, VT_STR, len(v))
            for s in v: out += _s(s)
        elif kind == "arr_i32":
            out += struct.pack("<IIQ", VT_ARR, VT_I32, len(v)) + np.asarray(v, "<i4").tobytes()
        else:
            raise ValueError(kind)
    offs, at = [], 0
    for name, dims, t, data in tensors:
        offs.append(at)
        at += (len(data) + alignment - 1) // alignment * alignment
    for (name, dims, t, data), off in zip(tensors, offs):
        out += _s(name) + struct.pack("<I", len(dims))
        for d in dims: out += struct.pack("<Q", d)
        out += struct.pack("<IQ", t, off)
    out += b"\0" * ((-len(out)) % alignment)
    data_off = len(out)
    for (name, dims, t, data), off in zip(tensors, offs):
        assert len(out) == data_off + off
        out += bytes(data)
        out += b"\0" * ((-len(data)) % alignment)
    with open(path, "wb") as f:
        f.write(out)
    return data_off, offs
