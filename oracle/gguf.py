"""TEST ORACLE for the GGUF container step (not product code: only tests/ may import this).

A plain-Python restatement of the reference's GGUF reader, src/gguf/mod.rs:
  magic / version check            :182-190
  key/value section                :192-202, value decoding :256-303
  tensor directory                 :204-215
  data section offset (align 32)   :217
  tensor_view (name lookup, size)  :237-254, with DType::storage_size src/tensor/mod.rs:36-93
and a small writer of the same format for building test files.

Pinned by tests/golden/tiny.gguf, a file written by the gguf-py package (the format's own Python
implementation) with tests/golden/make_gguf_fixture.py, and by that script's record of what
gguf-py's reader returns for it (tests/golden/tiny_gguf_expected.json)."""
from __future__ import annotations

import struct
from typing import Dict, List, Sequence, Tuple

import numpy as np

GGUF_MAGIC = 0x46554747
ALIGNMENT = 32

# GGUF type id -> (elements per block, bytes per block), src/tensor/mod.rs:36-86 and :96-130
BLOCK_LAYOUT = {0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 9: (32, 40),
                10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292),
                16: (256, 66), 17: (256, 74), 18: (256, 98), 19: (256, 50), 20: (32, 18), 21: (256, 110),
                22: (256, 82), 23: (32, 36), 24: (1, 1), 25: (1, 2), 26: (1, 4), 27: (1, 8), 28: (1, 8),
                29: (256, 56), 30: (1, 2)}

# metadata value type -> struct format (src/gguf/mod.rs:256-273)
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}
T_STRING, T_ARRAY, T_BOOL = 8, 9, 7


class GgufFormatError(ValueError):
    pass


def storage_size(dtype: int, n_elements: int) -> int:
    """DType::storage_size, src/tensor/mod.rs:89-93."""
    be, bb = BLOCK_LAYOUT[dtype]
    if n_elements % be:
        raise GgufFormatError(f"element count {n_elements} not divisible by block size {be}")
    return n_elements // be * bb


class _Reader:
    """src/gguf/mod.rs:119-166."""

    def __init__(self, buf: bytes):
        self.buf, self.pos = buf, 0

    def take(self, fmt: str):
        n = struct.calcsize(fmt)
        if self.pos + n > len(self.buf):
            raise GgufFormatError("file ends inside the GGUF directory")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += n
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GgufFormatError("file ends inside the GGUF directory")
        raw = self.buf[self.pos:self.pos + n]
        self.pos += n
        try:
            return raw.decode("utf-8")
        except UnicodeDecodeError:
            raise GgufFormatError("invalid UTF-8 in string")


def _read_value(r: _Reader):
    """Returns (type, elem_type or None, python value); src/gguf/mod.rs:256-303."""
    t = r.take("<I")
    if t == T_STRING:
        return t, None, r.string()
    if t == T_ARRAY:
        et = r.take("<I")
        n = r.take("<Q")
        if et == T_STRING:
            return t, et, [r.string() for _ in range(n)]
        if et not in _SCALAR:
            raise GgufFormatError(f"unknown metadata type: {et}")
        vals = [r.take(_SCALAR[et]) for _ in range(n)]
        return t, et, [bool(v) for v in vals] if et == T_BOOL else vals
    if t not in _SCALAR:
        raise GgufFormatError(f"unknown metadata type: {t}")
    v = r.take(_SCALAR[t])
    return t, None, bool(v) if t == T_BOOL else v


def parse(buf: bytes) -> dict:
    """GgufFile::open on the file's bytes (src/gguf/mod.rs:167-218).  Returns
    {version, metadata: {key: (type, elem_type, value)}, tensors: [{name, shape, dtype, offset, nbytes}], data_offset}."""
    r = _Reader(buf)
    magic = r.take("<I")
    if magic != GGUF_MAGIC:
        raise GgufFormatError(f"invalid GGUF magic: 0x{magic:08x}")
    version = r.take("<I")
    if version < 2 or version > 3:
        raise GgufFormatError(f"unsupported GGUF version: {version}")
    n_tensors, n_kv = r.take("<Q"), r.take("<Q")
    metadata: Dict[str, Tuple[int, object, object]] = {}
    for _ in range(n_kv):
        key = r.string()
        metadata[key] = _read_value(r)           # a repeated key replaces the earlier one (HashMap insert, :201)
    tensors: List[dict] = []
    for _ in range(n_tensors):
        name = r.string()
        n_dims = r.take("<I")
        shape = [r.take("<Q") for _ in range(n_dims)]
        dtype = r.take("<I")
        if dtype not in BLOCK_LAYOUT:
            raise GgufFormatError(f"unknown dtype: {dtype}")
        offset = r.take("<Q")
        n = 1
        for d in shape:
            n *= d
        tensors.append({"name": name, "shape": shape, "dtype": dtype, "offset": offset, "nbytes": storage_size(dtype, n)})
    data_offset = (r.pos + ALIGNMENT - 1) & ~(ALIGNMENT - 1)
    return {"version": version, "metadata": metadata, "tensors": tensors, "data_offset": data_offset}


def tensor_bytes(buf: bytes, parsed: dict, name: str) -> bytes:
    """TensorView.data of tensor_view(name) (src/gguf/mod.rs:242-254): first entry of that name."""
    for t in parsed["tensors"]:
        if t["name"] == name:
            start = parsed["data_offset"] + t["offset"]
            return buf[start:start + t["nbytes"]]
    raise KeyError(f"tensor not found: {name}")


# ---- writer (test files only) -----------------------------------------------------------------------

def _w_string(s) -> bytes:
    raw = s if isinstance(s, bytes) else s.encode("utf-8")
    return struct.pack("<Q", len(raw)) + raw


def _w_value(t: int, v, et: int | None = None) -> bytes:
    if t == T_STRING:
        return struct.pack("<I", t) + _w_string(v)
    if t == T_ARRAY:
        head = struct.pack("<IIQ", t, et, len(v))
        if et == T_STRING:
            return head + b"".join(_w_string(x) for x in v)
        return head + b"".join(struct.pack(_SCALAR[et], x) for x in v)
    return struct.pack("<I", t) + struct.pack(_SCALAR[t], v)


def build(metadata: Sequence[Tuple[str, int, object, int | None]], tensors: Sequence[Tuple[str, Sequence[int], int, bytes]],
          version: int = 3, tensor_alignment: int = ALIGNMENT) -> bytes:
    """A GGUF file as bytes.  metadata: (key, type, value, elem_type); tensors: (name, shape, dtype, raw bytes),
    laid out in order, each at the next multiple of `tensor_alignment` inside the data section."""
    out = struct.pack("<IIQQ", GGUF_MAGIC, version, len(tensors), len(metadata))
    for key, t, v, et in metadata:
        out += _w_string(key) + _w_value(t, v, et)
    offsets, pos = [], 0
    for _name, _shape, _dt, raw in tensors:
        pos = (pos + tensor_alignment - 1) // tensor_alignment * tensor_alignment
        offsets.append(pos)
        pos += len(raw)
    for (name, shape, dt, _raw), off in zip(tensors, offsets):
        out += _w_string(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
        out += struct.pack("<IQ", dt, off)
    out += b"\0" * (-len(out) % ALIGNMENT)
    data = bytearray(pos)
    for (_n, _s, _d, raw), off in zip(tensors, offsets):
        data[off:off + len(raw)] = raw
    return out + bytes(data)


def as_python(value):
    """numpy scalars/arrays from the product's reader -> plain python, for comparisons."""
    if isinstance(value, np.ndarray):
        return value.tolist()
    if isinstance(value, np.generic):
        return value.item()
    return value
