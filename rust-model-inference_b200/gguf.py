"""GGUF v3 writer and a small reader.

The writer produces the synthetic Qwen3-architecture checkpoints the benchmarks and
parity tests load (no model files exist offline).  The reader follows the parse order of
the reference loader (src/core/loader.rs:211-320: magic, version 2..3, tensor count, KV
count, KV table, tensor table, data offset padded to `general.alignment`, default 32) and
is what the tests use to hand raw tensor bytes to the CPU oracle.  The product's own
loader is the C++ one inside librmi_cuda.so (rmi_gguf_open); this file never feeds it.
"""
from __future__ import annotations

import mmap
import struct

import numpy as np

GGML_F32, GGML_F16, GGML_Q8_0, GGML_Q4_K = 0, 1, 8, 12
# src/core/tensor.rs:61-81 type_traits: (block elements, block bytes)
TYPE_TRAITS = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144)}
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_SCALAR_FMT = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i",
               T_F32: "<f", T_BOOL: "<B", T_U64: "<Q", T_I64: "<q", T_F64: "<d"}
ALIGN = 32


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, vtype: int, value) -> bytes:
    out = _s(key) + struct.pack("<i", vtype)
    if vtype == T_STR:
        return out + _s(value)
    if vtype == T_ARR:
        etype, items = value
        out += struct.pack("<iQ", etype, len(items))
        for it in items:
            out += _s(it) if etype == T_STR else struct.pack(_SCALAR_FMT[etype], it)
        return out
    return out + struct.pack(_SCALAR_FMT[vtype], value)


def nbytes(ggml_type: int, n_elements: int) -> int:
    be, bb = TYPE_TRAITS[ggml_type]
    return (n_elements + be - 1) // be * bb


def write_gguf(path: str, metadata: list, tensors: list) -> None:
    """metadata: [(key, vtype, value)], tensors: [(name, dims(list, dims[0] = row length),
    ggml_type, uint8 ndarray)]."""
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(metadata))
    for key, vtype, value in metadata:
        head += _kv(key, vtype, value)
    offs, off = [], 0
    for name, dims, gtype, data in tensors:
        n_el = int(np.prod(dims))
        assert data.nbytes == nbytes(gtype, n_el), (name, data.nbytes, nbytes(gtype, n_el))
        offs.append(off)
        off = (off + data.nbytes + ALIGN - 1) // ALIGN * ALIGN
    for (name, dims, gtype, _), o in zip(tensors, offs):
        head += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<iQ", gtype, o)
    pad = (-len(head)) % ALIGN
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        pos = 0
        for (_, _, _, data), o in zip(tensors, offs):
            if o > pos:
                f.write(b"\0" * (o - pos))
                pos = o
            f.write(np.ascontiguousarray(data).view(np.uint8).reshape(-1).tobytes())
            pos += data.nbytes


class GGUFFile:
    """mmap-backed reader: .metadata dict, .tensors {name: (dims, type, uint8 view)}."""

    def __init__(self, path: str):
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        buf = self._mm
        self._pos = 0

        def rd(fmt):
            v = struct.unpack_from(fmt, buf, self._pos)
            self._pos += struct.calcsize(fmt)
            return v[0] if len(v) == 1 else v

        def rstr():
            n = rd("<Q")
            if self._pos + n > len(buf):
                raise ValueError("string exceeds GGUF data")
            s = bytes(buf[self._pos:self._pos + n]).decode()
            self._pos += n
            return s

        def rval(t):
            if t == T_STR:
                return rstr()
            if t == T_ARR:
                et, n = rd("<i"), rd("<Q")
                return [rval(et) for _ in range(n)]
            if t not in _SCALAR_FMT:
                raise ValueError(f"Unknown meta value type: {t}")
            return rd(_SCALAR_FMT[t])

        if bytes(buf[:4]) != b"GGUF":
            raise ValueError("Invalid GGUF magic")
        self._pos = 4
        self.version = rd("<I")
        if not 2 <= self.version <= 3:
            raise ValueError(f"Unsupported GGUF version: {self.version}")
        n_t, n_kv = rd("<Q"), rd("<Q")
        self.metadata = {}
        for _ in range(n_kv):
            k = rstr()
            self.metadata[k] = rval(rd("<i"))
        infos = []
        for _ in range(n_t):
            name = rstr()
            nd = rd("<I")
            dims = [rd("<Q") for _ in range(nd)]
            infos.append((name, dims, rd("<i"), rd("<Q")))
        align = int(self.metadata.get("general.alignment", ALIGN))
        if align == 0:
            raise ValueError("GGUF alignment must be nonzero")
        self.data_offset = (self._pos + align - 1) // align * align
        self.tensors = {}
        whole = np.frombuffer(buf, np.uint8)
        for name, dims, gtype, off in infos:
            n = nbytes(gtype, int(np.prod(dims)))
            s = self.data_offset + off
            if s + n > len(buf):
                raise ValueError(f"tensor {name} exceeds GGUF data")
            self.tensors[name] = (dims, gtype, whole[s:s + n])

    def tensor(self, name: str) -> np.ndarray:
        return self.tensors[name][2]
