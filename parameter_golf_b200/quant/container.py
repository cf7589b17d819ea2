"""Artifact containers: PGRS tensor file, PGPG per-group compression, zstd through ``libzstd.so.1``.

Byte formats (all little-endian):

* **PGRS v1** (``parameter-golf-rs/crates/pg-quant/src/serialize.rs:6-20,60-99``): ``"PGRS"``, u32 version=1,
  u32 num_tensors; per tensor u32 name_len, UTF-8 name, u32 ndim, ndim x u32 dims, u8 dtype code
  (BF16=0, F16=1, F32=2, I8=3, I32=4, U16=5, U32=6), u32 data_len, data, u32 CRC32(data) (IEEE);
  then u32 metadata_len and the metadata JSON.
* **PGPG** (``pg-quant/src/compress.rs:33-53``): ``"PGPG"``, u32 version=1, u64 raw_len, u32 chunk_bytes,
  u32 group_count, then per group u32 raw_len, u32 comp_len, one zstd frame.
* Sniffing (``compress.rs:101-109``): ``PGPG`` -> per-group, ``PGRS`` -> raw, the xz magic -> one xz stream (``lzma9``,
  which the reference declares but does not write), anything else -> one zstd frame.

The image ships the zstd runtime library without headers or Python bindings, so the five entry
points used here are declared through ctypes.
"""
from __future__ import annotations

import ctypes
import struct
import zlib
from dataclasses import dataclass
from typing import List, Tuple

import numpy as np

DTYPE_CODES = {"bf16": 0, "f16": 1, "f32": 2, "i8": 3, "i32": 4, "u16": 5, "u32": 6, "f8e4m3": 7}
CODE_NAMES = {v: k for k, v in DTYPE_CODES.items()}
DTYPE_SIZES = {"bf16": 2, "f16": 2, "f32": 4, "i8": 1, "i32": 4, "u16": 2, "u32": 4, "f8e4m3": 1}
DEFAULT_CHUNK_BYTES = 1 << 20


class ArtifactError(ValueError):
    pass


@dataclass
class TensorRecord:
    name: str
    dims: Tuple[int, ...]
    dtype: str          # key of DTYPE_CODES
    data: bytes         # raw payload (bit-packed payloads are shorter than prod(dims)*itemsize)


# ---- native primitives ----------------------------------------------------------------------------
_native_mod = None


def _native():
    """The C++ implementations of bit packing, CRC-32 and the PGRS container (``csrc/artifact.cpp``), or ``None`` when the
    extension has not been built; the NumPy forms below are the specification they are tested against."""
    global _native_mod
    if _native_mod is None:
        try:
            from ..ops import native
            _native_mod = native.load_raw() if native.available() else False
        except Exception:
            _native_mod = False
    return _native_mod or None


# ---- zstd via ctypes ------------------------------------------------------------------------------
_zstd = None


def _lib():
    global _zstd
    if _zstd is None:
        lib = ctypes.CDLL("libzstd.so.1")
        lib.ZSTD_compressBound.restype = ctypes.c_size_t
        lib.ZSTD_compressBound.argtypes = [ctypes.c_size_t]
        lib.ZSTD_compress.restype = ctypes.c_size_t
        lib.ZSTD_compress.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        lib.ZSTD_decompress.restype = ctypes.c_size_t
        lib.ZSTD_decompress.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t]
        lib.ZSTD_getFrameContentSize.restype = ctypes.c_ulonglong
        lib.ZSTD_getFrameContentSize.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
        lib.ZSTD_isError.restype = ctypes.c_uint
        lib.ZSTD_isError.argtypes = [ctypes.c_size_t]
        _zstd = lib
    return _zstd


def zstd_compress(data: bytes, level: int = 22) -> bytes:
    lib = _lib()
    cap = lib.ZSTD_compressBound(len(data))
    dst = ctypes.create_string_buffer(cap)
    n = lib.ZSTD_compress(dst, cap, data, len(data), level)
    if lib.ZSTD_isError(n):
        raise ArtifactError("zstd compression failed")
    return dst.raw[:n]


def zstd_decompress(data: bytes) -> bytes:
    lib = _lib()
    size = lib.ZSTD_getFrameContentSize(data, len(data))
    if size in (0xFFFFFFFFFFFFFFFF, 0xFFFFFFFFFFFFFFFE):
        raise ArtifactError("not a zstd frame with a known content size")
    dst = ctypes.create_string_buffer(max(int(size), 1))
    n = lib.ZSTD_decompress(dst, int(size), data, len(data))
    if lib.ZSTD_isError(n) or n != size:
        raise ArtifactError("zstd decompression failed")
    return dst.raw[:n]


# ---- PGRS -------------------------------------------------------------------------------------------

def write_pgrs(tensors: List[TensorRecord], metadata: str, native: bool = True) -> bytes:
    nat = _native() if native else None
    if nat is not None:
        return nat.write_pgrs([(t.name, [int(d) for d in t.dims], DTYPE_CODES[t.dtype], bytes(t.data)) for t in tensors], metadata)
    out = bytearray(b"PGRS")
    out += struct.pack("<II", 1, len(tensors))
    for t in tensors:
        name = t.name.encode("utf-8")
        out += struct.pack("<I", len(name)) + name
        out += struct.pack("<I", len(t.dims)) + b"".join(struct.pack("<I", int(d)) for d in t.dims)
        out += struct.pack("<B", DTYPE_CODES[t.dtype])
        out += struct.pack("<I", len(t.data)) + t.data
        out += struct.pack("<I", zlib.crc32(t.data) & 0xFFFFFFFF)
    meta = metadata.encode("utf-8")
    out += struct.pack("<I", len(meta)) + meta
    return bytes(out)


def read_pgrs(buf: bytes, native: bool = True) -> Tuple[List[TensorRecord], str]:
    nat = _native() if native else None
    if nat is not None:
        try:
            recs, meta = nat.read_pgrs(bytes(buf))
        except RuntimeError as e:
            raise ArtifactError(str(e)) from None
        return [TensorRecord(n, tuple(d), CODE_NAMES[c], data) for n, d, c, data in recs], meta
    if len(buf) < 12 or buf[:4] != b"PGRS":
        raise ArtifactError("not a PGRS file")
    pos = 4

    def take(n):
        nonlocal pos
        if pos + n > len(buf):
            raise ArtifactError("truncated PGRS file")
        b = buf[pos:pos + n]
        pos += n
        return b

    def u32():
        return struct.unpack("<I", take(4))[0]

    version, count = u32(), u32()
    if version != 1:
        raise ArtifactError(f"unsupported PGRS version {version}")
    tensors = []
    for _ in range(count):
        name = take(u32()).decode("utf-8")
        ndim = u32()
        dims = tuple(u32() for _ in range(ndim))
        code = take(1)[0]
        if code not in CODE_NAMES:
            raise ArtifactError(f"tensor {name}: unknown dtype code {code}")
        data = bytes(take(u32()))
        crc = u32()
        if zlib.crc32(data) & 0xFFFFFFFF != crc:
            raise ArtifactError(f"tensor {name}: CRC mismatch (corrupted artifact)")
        tensors.append(TensorRecord(name, dims, CODE_NAMES[code], data))
    metadata = take(u32()).decode("utf-8")
    return tensors, metadata


# ---- PGPG + sniffing ------------------------------------------------------------------------------------

def compress_pergroup(raw: bytes, chunk_bytes: int = DEFAULT_CHUNK_BYTES, level: int = 22) -> bytes:
    chunks = [raw[i:i + chunk_bytes] for i in range(0, len(raw), chunk_bytes)] or [b""]
    out = bytearray(b"PGPG")
    out += struct.pack("<IQII", 1, len(raw), chunk_bytes, len(chunks))
    for c in chunks:
        z = zstd_compress(c, level)
        out += struct.pack("<II", len(c), len(z)) + z
    return bytes(out)


def decompress_pergroup(buf: bytes) -> bytes:
    version, raw_len, _chunk, groups = struct.unpack_from("<IQII", buf, 4)
    if version != 1:
        raise ArtifactError(f"unsupported PGPG version {version}")
    pos, out = 24, bytearray()
    for _ in range(groups):
        r, c = struct.unpack_from("<II", buf, pos)
        pos += 8
        part = zstd_decompress(buf[pos:pos + c]) if r else b""
        if len(part) != r:
            raise ArtifactError("PGPG group length mismatch")
        out += part
        pos += c
    if len(out) != raw_len:
        raise ArtifactError("PGPG total length mismatch")
    return bytes(out)


def compress_payload(raw: bytes, mode: str) -> bytes:
    if mode == "none":
        return raw
    if mode == "zstd22":
        return zstd_compress(raw, 22)
    if mode == "lzma9":        # one xz stream, preset 9 (the reference declares this mode and rejects it, export.rs:195-198)
        import lzma
        return lzma.compress(raw, format=lzma.FORMAT_XZ, preset=9 | lzma.PRESET_EXTREME)
    if mode == "pergroup":
        return compress_pergroup(raw)
    raise ArtifactError(f"unsupported compression mode {mode!r}")


def decompress_payload(buf: bytes) -> bytes:
    if buf[:4] == b"PGPG":
        return decompress_pergroup(buf)
    if buf[:4] == b"PGRS":
        return buf
    if buf[:6] == b"\xfd7zXZ\x00":
        import lzma
        try:
            return lzma.decompress(buf, format=lzma.FORMAT_XZ)
        except lzma.LZMAError as e:
            raise ArtifactError(f"xz decompression failed: {e}") from e
    return zstd_decompress(buf)


# ---- bit packing --------------------------------------------------------------------------------------

def pack_bits(q: np.ndarray, bits: int, native: bool = True) -> bytes:
    """LSB-first little-endian bit stream of ``q - qmin`` (unsigned, ``bits`` wide), elements back to
    back with no row padding (``pg-quant/src/export.rs:542-558``)."""
    nat = _native() if native else None
    if nat is not None and 2 <= bits <= 8 and q.size and int(np.abs(q).max()) < 128:
        try:
            return nat.pack_bits(np.ascontiguousarray(q.reshape(-1).astype(np.int8)), bits)
        except RuntimeError as e:
            raise ArtifactError(str(e)) from None
    qmin = -(1 << (bits - 1))
    e = (q.astype(np.int32).reshape(-1) - qmin).astype(np.uint32)
    if e.size and int(e.max()) >= (1 << bits):
        raise ArtifactError("quantised value out of range for bit width")
    b = ((e[:, None] >> np.arange(bits, dtype=np.uint32)[None, :]) & 1).astype(np.uint8).reshape(-1)
    return np.packbits(b, bitorder="little").tobytes()


def unpack_bits(data: bytes, count: int, bits: int, native: bool = True) -> np.ndarray:
    nat = _native() if native else None
    if nat is not None and 2 <= bits <= 8:
        try:
            return nat.unpack_bits(bytes(data), count, bits).astype(np.int32)
        except RuntimeError as e:
            raise ArtifactError(str(e)) from None
    qmin = -(1 << (bits - 1))
    need = (count * bits + 7) // 8
    if len(data) < need:
        raise ArtifactError("packed tensor is shorter than its shape requires")
    b = np.unpackbits(np.frombuffer(data, dtype=np.uint8, count=need), bitorder="little")[: count * bits]
    w = (1 << np.arange(bits, dtype=np.int32))
    return (b.reshape(count, bits).astype(np.int32) * w[None, :]).sum(1).astype(np.int32) + qmin
