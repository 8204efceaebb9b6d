"""BIDMat matrix files, as the reference's corpora and checkpoints use them.

The reference reads its training text with ``loadMat`` (``train%05d.imat.lz4``:
2 x N int32, row 0 word ids, row 1 sentence ids; scripts/getw2vdata.ssc:8-48,
scripts/testword2vec.ssc:3-5) and writes ``modelmat%02d.lz4`` per model matrix
(models/Model.scala:245-263).  BIDMat is an un-vendored dependency; the dense
file layout is pinned by the reference's own C writers
(src/main/C/newparse/utils.cpp:350-362, 423-436, 484-509):

    int32 type, int32 nrows, int32 ncols, int32 nnz      little-endian
    nrows * ncols elements, column-major

``type`` 110 = int32, 120 = int64, 130 = float32, 140 = float64.  The extension
selects the compression of the whole stream: none, ``.gz`` (gzip, as
utils.cpp:300-341), or ``.lz4``: lz4-java's block stream.  That container is
restated from the library's published format and pinned by the one such file
in the BIDMach checkout (scripts/networks/modelmat_test.fmat.lz4, whose blocks
are stored raw: framing, checksum and end mark are pinned by it, the
LZ4-compressed block method by interoperation with another LZ4 implementation
in the tests): per block the 8 bytes
``LZ4Block``, a token byte (method 0x10 raw / 0x20 LZ4, or'ed with
``log2(blocksize) - 10``), int32 compressed length, int32 original length, int32
XXH32 checksum of the original bytes (seed 0x9747b28c, low 28 bits), then the
payload; a block of zero lengths ends the stream.

A 2 x N token matrix in column-major order is byte for byte the ``[N, 2]``
row-major int32 array the rest of this package uses for a minibatch source.
"""
from __future__ import annotations

import ctypes as C
import gzip
import os
import struct

import numpy as np

from . import _lib

_TYPES = {110: np.dtype("<i4"), 120: np.dtype("<i8"), 130: np.dtype("<f4"), 140: np.dtype("<f8")}
_CODES = {v: k for k, v in _TYPES.items()}

_MAGIC = b"LZ4Block"
_METHOD_RAW, _METHOD_LZ4 = 0x10, 0x20
_LEVEL_BASE = 10
_SEED = 0x9747B28C
_BLOCK = 1 << 16


def _u8(b) -> np.ndarray:
    return np.frombuffer(b, dtype=np.uint8)


def xxh32(data, seed: int = 0) -> int:
    a = _u8(data)
    return int(_lib.load().bidmach_xxh32(a.ctypes.data if a.size else None, a.size, seed))


def lz4_block_compress(data) -> bytes:
    lib = _lib.load()
    a = _u8(data)
    cap = lib.bidmach_lz4_compress_bound(a.size)
    out = np.empty(cap, np.uint8)
    n = lib.bidmach_lz4_compress(a.ctypes.data if a.size else None, a.size, out.ctypes.data, cap)
    if n < 0:
        raise RuntimeError("lz4 compression failed")
    return out[:n].tobytes()


def lz4_block_decompress(data, original_len: int) -> bytes:
    lib = _lib.load()
    a = _u8(data)
    out = np.empty(max(1, original_len), np.uint8)
    n = lib.bidmach_lz4_decompress(a.ctypes.data if a.size else None, a.size, out.ctypes.data, original_len)
    if n != original_len:
        raise ValueError("malformed LZ4 block")
    return out[:n].tobytes()


def lz4_stream_compress(raw: bytes, block_size: int = _BLOCK) -> bytes:
    level = max(0, (block_size - 1).bit_length() - _LEVEL_BASE)
    parts = []
    view = memoryview(raw)
    for lo in range(0, len(raw), block_size):
        chunk = view[lo: lo + block_size]
        check = xxh32(chunk, _SEED) & 0x0FFFFFFF
        comp = lz4_block_compress(chunk)
        if len(comp) >= len(chunk):
            method, payload = _METHOD_RAW, bytes(chunk)
        else:
            method, payload = _METHOD_LZ4, comp
        parts.append(_MAGIC + struct.pack("<BiiI", method | level, len(payload), len(chunk), check))
        parts.append(payload)
    parts.append(_MAGIC + struct.pack("<BiiI", _METHOD_RAW | level, 0, 0, 0))
    return b"".join(parts)


def lz4_stream_decompress(data: bytes) -> bytes:
    out = []
    at, n = 0, len(data)
    while at < n:
        if data[at: at + 8] != _MAGIC or at + 21 > n:
            raise ValueError("not an LZ4 block stream")
        token, clen, olen, check = struct.unpack_from("<BiiI", data, at + 8)
        at += 21
        if olen == 0 and clen == 0:
            if check != 0:
                raise ValueError("LZ4 block stream: bad end mark")
            break                      # end mark (a concatenated stream would start again; not supported)
        method = token & 0xF0
        if clen < 0 or olen < 0 or at + clen > n or olen > 1 << ((token & 0x0F) + _LEVEL_BASE):
            raise ValueError("LZ4 block stream: bad block header")
        payload = data[at: at + clen]
        at += clen
        if method == _METHOD_RAW:
            if clen != olen:
                raise ValueError("LZ4 block stream: raw block with two lengths")
            chunk = bytes(payload)
        elif method == _METHOD_LZ4:
            chunk = lz4_block_decompress(payload, olen)
        else:
            raise ValueError("LZ4 block stream: unknown compression method")
        h = xxh32(chunk, _SEED)
        if check not in (h & 0x0FFFFFFF, h):
            raise ValueError("LZ4 block stream: checksum mismatch")
        out.append(chunk)
    return b"".join(out)


def _read_all(fname: str) -> bytes:
    with open(fname, "rb") as f:
        data = f.read()
    if fname.endswith(".lz4"):
        return lz4_stream_decompress(data)
    if fname.endswith(".gz"):
        return gzip.decompress(data)
    return data


def peekShape(fname: str):
    """(nrows, ncols) from the header, reading as little of the file as the compression allows."""
    if fname.endswith(".gz"):
        with gzip.open(fname, "rb") as f:
            head = f.read(16)
    elif fname.endswith(".lz4"):
        with open(fname, "rb") as f:
            first = f.read(21)
            if first[:8] != _MAGIC or len(first) < 21:
                raise ValueError("%s: not an LZ4 block stream" % fname)
            clen = struct.unpack_from("<i", first, 9)[0]
            head = lz4_stream_decompress(first + f.read(max(0, clen)) + _MAGIC + struct.pack("<BiiI", _METHOD_RAW, 0, 0, 0))[:16]
    else:
        with open(fname, "rb") as f:
            head = f.read(16)
    if len(head) < 16:
        raise ValueError("%s: too short for a matrix header" % fname)
    _t, nrows, ncols, _nnz = struct.unpack_from("<iiii", head, 0)
    return nrows, ncols


def loadMat(fname: str) -> np.ndarray:
    """The dense matrix stored in ``fname`` as a Fortran-ordered ``[nrows, ncols]``
    array (``.T`` of it is the C-ordered ``[ncols, nrows]`` view of the same bytes)."""
    raw = _read_all(fname)
    if len(raw) < 16:
        raise ValueError("%s: too short for a matrix header" % fname)
    mtype, nrows, ncols, _nnz = struct.unpack_from("<iiii", raw, 0)
    if mtype not in _TYPES:
        raise NotImplementedError("%s: matrix type %d (only dense int/long/float/double)" % (fname, mtype))
    dt = _TYPES[mtype]
    need = 16 + nrows * ncols * dt.itemsize
    if nrows < 0 or ncols < 0 or len(raw) < need:
        raise ValueError("%s: %d x %d matrix does not fit %d bytes" % (fname, nrows, ncols, len(raw)))
    return np.frombuffer(raw, dtype=dt, count=nrows * ncols, offset=16).reshape((nrows, ncols), order="F")


def saveMat(fname: str, a) -> None:
    """Writes a 1-D (one column) or 2-D array; the extension picks the compression."""
    if hasattr(a, "detach"):
        a = a.detach().cpu().numpy()
    a = np.asarray(a)
    if a.ndim == 1:
        a = a.reshape(-1, 1)
    if a.ndim != 2:
        raise ValueError("only matrices")
    dt = a.dtype.newbyteorder("<") if a.dtype.byteorder == ">" else a.dtype
    if np.dtype(dt) not in _CODES:
        raise NotImplementedError("dtype %s" % a.dtype)
    nrows, ncols = a.shape
    raw = struct.pack("<iiii", _CODES[np.dtype(dt)], nrows, ncols, nrows * ncols if _is_vec(a) else 0) + \
        np.asfortranarray(a, dtype=dt).tobytes(order="F")
    if fname.endswith(".lz4"):
        raw = lz4_stream_compress(raw)
    elif fname.endswith(".gz"):
        raw = gzip.compress(raw, compresslevel=6)
    parent = os.path.dirname(fname)
    if parent:
        os.makedirs(parent, exist_ok=True)
    with open(fname, "wb") as f:
        f.write(raw)


def _is_vec(a) -> bool:
    # the reference's vector writers store nnz = nrows, its matrix writers 0
    # (utils.cpp:356-357 against 459-460); readers ignore the field for dense types
    return a.shape[1] == 1


def loadTokens(fname: str) -> np.ndarray:
    """A corpus file (2 x N int32: word ids over sentence ids) as the ``[N, 2]``
    minibatch layout of this package; no bytes are moved."""
    m = loadMat(fname)
    if m.dtype != np.int32 or m.shape[0] != 2:
        raise ValueError("%s: expected a 2 x N int32 matrix, found %s %s" % (fname, m.shape, m.dtype))
    return m.T


def saveTokens(fname: str, tokens) -> None:
    t = np.ascontiguousarray(tokens, dtype=np.int32)
    if t.ndim != 2 or t.shape[1] != 2:
        raise ValueError("tokens must be [N, 2]")
    saveMat(fname, t.T)
