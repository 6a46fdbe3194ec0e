"""Read quantized tensors straight out of a GGUF file, so that converted models can be fed to the library
without the reference's Go loader (its reader: convert/gguf/gguf.go:73-182).

GGUF v2/v3, little-endian: magic "GGUF", u32 version, u64 tensor count, u64 key/value count; the key/value
section; the tensor table (name, u32 n_dims, u64 dims innermost first, u32 ggml type, u64 offset into the data
section); the data section starts at the next multiple of `general.alignment` (default 32). A matrix has
dims = [k, rows]; an expert bank [k, rows, n_expert]. The file is memory-mapped: `tensor_bytes` returns a view,
nothing is copied until it is uploaded.
"""
from __future__ import annotations

import mmap
import struct

import numpy as np

from ._lib import BLOCK, F16, F32, BF16, MXFP4, Q4_K, Q8_0

MAGIC = 0x46554747          # "GGUF"
MAX_DIMS = 4
# key/value types of the format
_U8, _I8, _U16, _I16, _U32, _I32, _F32, _BOOL, _STR, _ARR, _U64, _I64, _F64 = range(13)
_SCALAR = {_U8: "<B", _I8: "<b", _U16: "<H", _I16: "<h", _U32: "<I", _I32: "<i", _F32: "<f", _BOOL: "<?", _U64: "<Q",
           _I64: "<q", _F64: "<d"}
_FLOAT_BYTES = {F32: 4, F16: 2, BF16: 2}


class GGUFError(ValueError):
    pass


class _Cursor:
    def __init__(self, buf):
        self.b, self.o = buf, 0

    def take(self, fmt):
        n = struct.calcsize(fmt)
        if self.o + n > len(self.b):
            raise GGUFError(f"truncated at byte {self.o}")
        v = struct.unpack_from(fmt, self.b, self.o)[0]
        self.o += n
        return v

    def string(self):
        n = self.take("<Q")
        if n > len(self.b) - self.o:
            raise GGUFError(f"string of {n} bytes at byte {self.o} runs past the end of the file")
        s = bytes(self.b[self.o:self.o + n])
        self.o += n
        return s.decode("utf-8", errors="replace")

    def value(self, vt, depth=0):
        if vt in _SCALAR:
            return self.take(_SCALAR[vt])
        if vt == _STR:
            return self.string()
        if vt == _ARR:
            if depth > 2:
                raise GGUFError("arrays nested too deep")
            et, n = self.take("<I"), self.take("<Q")
            if n > len(self.b) - self.o:          # every element takes at least one byte
                raise GGUFError(f"array of {n} elements at byte {self.o} cannot fit the file")
            return [self.value(et, depth + 1) for _ in range(n)]
        raise GGUFError(f"unknown key/value type {vt}")


def tensor_nbytes(t: int, dims) -> int:
    """Bytes of a tensor of ggml type t; the innermost dim must tile the type's block."""
    n = 1
    for d in dims:
        n *= int(d)
    if t in _FLOAT_BYTES:
        return n * _FLOAT_BYTES[t]
    if t not in BLOCK:
        raise GGUFError(f"ggml type {t} is not one this library sizes")
    be, bb = BLOCK[t]
    if not dims or dims[0] % be:
        raise GGUFError(f"innermost dim {dims[0] if dims else None} does not tile {be}-element blocks")
    return n // be * bb


class GGUFReader:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        try:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError as e:                   # empty file
            self._f.close()
            raise GGUFError(f"{path}: {e}") from None
        try:
            self._parse()
        except Exception:
            self.close()
            raise

    def _parse(self):
        c = _Cursor(self._mm)
        if c.take("<I") != MAGIC:
            raise GGUFError(f"{self.path}: not a GGUF file")
        self.version = c.take("<I")
        if self.version not in (2, 3):
            raise GGUFError(f"{self.path}: unsupported version {self.version} (want 2 or 3)")
        n_tensors, n_kv = c.take("<Q"), c.take("<Q")
        left = len(self._mm) - c.o
        if n_kv * 13 > left or n_tensors * 25 > left:    # smallest possible entries: refuse before allocating
            raise GGUFError(f"{self.path}: {n_tensors} tensors / {n_kv} keys cannot fit {left} bytes")
        self.kv = {}
        for i in range(n_kv):
            key = c.string()
            self.kv[key] = c.value(c.take("<I"))
        self.alignment = int(self.kv.get("general.alignment", 32))
        if self.alignment < 1 or self.alignment & (self.alignment - 1):
            raise GGUFError(f"{self.path}: general.alignment {self.alignment} is not a power of two")
        self.tensors = {}
        for i in range(n_tensors):
            name = c.string()
            nd = c.take("<I")
            if nd > MAX_DIMS:
                raise GGUFError(f"{self.path}: tensor {name!r} has {nd} dimensions (max {MAX_DIMS})")
            dims = [c.take("<Q") for _ in range(nd)]
            t, off = c.take("<I"), c.take("<Q")
            if name in self.tensors:
                raise GGUFError(f"{self.path}: duplicate tensor name {name!r}")
            self.tensors[name] = {"type": t, "dims": dims, "offset": off}
        self.data_start = (c.o + self.alignment - 1) & ~(self.alignment - 1)
        if self.data_start > len(self._mm):
            raise GGUFError(f"{self.path}: the data section starts past the end of the file")
        for name, info in self.tensors.items():
            try:
                info["nbytes"] = tensor_nbytes(info["type"], info["dims"])
            except GGUFError:
                info["nbytes"] = None              # a type this library does not size: listed, not readable
                continue
            if info["offset"] % self.alignment:
                raise GGUFError(f"{self.path}: tensor {name!r} sits at an unaligned offset {info['offset']}")
            if self.data_start + info["offset"] + info["nbytes"] > len(self._mm):
                raise GGUFError(f"{self.path}: tensor {name!r} runs past the end of the file")

    # ------------------------------------------------------------------ access
    def tensor_bytes(self, name: str) -> np.ndarray:
        """The raw ggml bytes of a tensor as a read-only uint8 view of the mapped file."""
        info = self.tensors[name]
        if info["nbytes"] is None:
            raise GGUFError(f"tensor {name!r} has ggml type {info['type']}, which this library does not size")
        start = self.data_start + info["offset"]
        return np.frombuffer(self._mm, dtype=np.uint8, count=info["nbytes"], offset=start)

    def matrix_shape(self, name: str):
        """(n_expert, rows, k) of a 2-D matrix or a 3-D expert bank."""
        dims = self.tensors[name]["dims"]
        if len(dims) == 2:
            return 1, int(dims[1]), int(dims[0])
        if len(dims) == 3:
            return int(dims[2]), int(dims[1]), int(dims[0])
        raise GGUFError(f"tensor {name!r} has {len(dims)} dimensions: not a matrix or an expert bank")

    def upload(self, dev, name: str):
        """Upload a Q4_K / Q8_0 / MXFP4 matrix or bank to `dev` (jitllm_b200.Device) and return its Weight handle."""
        info = self.tensors[name]
        if info["type"] not in (Q4_K, Q8_0, MXFP4):
            raise GGUFError(f"tensor {name!r} has ggml type {info['type']}: the device path serves Q4_K, Q8_0 and MXFP4")
        n_expert, rows, k = self.matrix_shape(name)
        return dev.Upload(info["type"], self.tensor_bytes(name), rows, k, n_expert)

    def close(self):
        mm, self._mm = getattr(self, "_mm", None), None
        if mm is not None:
            try:
                mm.close()
            except BufferError:                    # a view handed out by tensor_bytes is still alive
                pass
        if self._f:
            self._f.close()
            self._f = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_gguf(path: str, kv: dict, tensors: dict, alignment: int = 32, version: int = 3) -> None:
    """Minimal writer (tests and synthetic models): tensors = {name: (ggml_type, dims innermost first, bytes)};
    kv values may be int (u32), float (f32), bool, str, or a list of one of those."""
    def enc_str(s):
        b = s.encode("utf-8")
        return struct.pack("<Q", len(b)) + b

    def enc_val(v):
        if isinstance(v, bool):
            return _BOOL, struct.pack("<?", v)
        if isinstance(v, int):
            return _U32, struct.pack("<I", v)
        if isinstance(v, float):
            return _F32, struct.pack("<f", v)
        if isinstance(v, str):
            return _STR, enc_str(v)
        if isinstance(v, (list, tuple)):
            if not v:
                return _ARR, struct.pack("<IQ", _U32, 0)
            et, _ = enc_val(v[0])
            return _ARR, struct.pack("<IQ", et, len(v)) + b"".join(enc_val(e)[1] for e in v)
        raise TypeError(type(v))

    kv = dict(kv)
    if alignment != 32:
        kv["general.alignment"] = alignment
    head = struct.pack("<IIQQ", MAGIC, version, len(tensors), len(kv))
    for key, v in kv.items():
        vt, payload = enc_val(v)
        head += enc_str(key) + struct.pack("<I", vt) + payload
    off, table, blobs = 0, b"", []
    for name, (t, dims, data) in tensors.items():
        data = bytes(data)
        table += enc_str(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        table += struct.pack("<IQ", t, off)
        blobs.append((off, data))
        off = (off + len(data) + alignment - 1) // alignment * alignment
    head += table
    pad = (-len(head)) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        pos = 0
        for o, data in blobs:
            f.write(b"\0" * (o - pos) + data)
            pos = o + len(data)
