"""BIDMat matrix files (raw, .gz, .lz4), the byte codecs behind them, and the
file-backed minibatch source.  CPU only: the codecs are host code of the library."""
import gzip
import struct

import numpy as np
import pytest


def test_xxh32_known_answers():
    """Published XXH32 test values (seed 0 unless noted)."""
    from bidmach_b200 import matio
    assert matio.xxh32(b"") == 0x02CC5D05
    assert matio.xxh32(b"a") == 0x550D7456
    assert matio.xxh32(b"abc") == 0x32D153FF
    assert matio.xxh32(b"Nobody inspects the spammish repetition") == 0xE2293B2F
    assert matio.xxh32(b"", 2654435761) == 0x36B78AE7


def _cases():
    rng = np.random.default_rng(0)
    return [b"", b"a", b"hello hello hello hello hello hello", bytes(1000),
            rng.integers(0, 4, 100_000, dtype=np.uint8).tobytes(),
            rng.integers(0, 256, 70_000, dtype=np.uint8).tobytes(),
            np.arange(50_000, dtype=np.int32).tobytes(),
            (b"abcd" * 5000) + b"xyz"]


@pytest.mark.parametrize("k", range(8))
def test_lz4_block_round_trip_and_interoperates_with_another_implementation(k):
    from bidmach_b200 import matio
    data = _cases()[k]
    comp = matio.lz4_block_compress(data)
    assert matio.lz4_block_decompress(comp, len(data)) == data
    pa = pytest.importorskip("pyarrow")
    try:
        codec = pa.Codec("lz4_raw")
    except Exception:
        pytest.skip("this pyarrow has no raw LZ4 codec")
    if data:
        assert codec.decompress(comp, decompressed_size=len(data), asbytes=True) == data
        assert matio.lz4_block_decompress(codec.compress(data, asbytes=True), len(data)) == data


def test_lz4_block_decoder_rejects_malformed_input():
    from bidmach_b200 import matio
    good = matio.lz4_block_compress(b"hello hello hello hello hello hello")
    with pytest.raises(ValueError):
        matio.lz4_block_decompress(good[:-3], 35)          # truncated
    with pytest.raises(ValueError):
        matio.lz4_block_decompress(good, 20)               # more output than announced
    with pytest.raises(ValueError):
        matio.lz4_block_decompress(b"\x10a\x05\x00", 10)    # offset reaches before the output
    with pytest.raises(ValueError):
        matio.lz4_stream_decompress(b"LZ4Blocc" + bytes(13))


def test_lz4_stream_layout():
    """Block header: magic, token, compressed length, original length, 28-bit checksum;
    incompressible blocks are stored raw; a zero block ends the stream."""
    from bidmach_b200 import matio
    rng = np.random.default_rng(1)
    data = bytes(70_000) + rng.integers(0, 256, 70_000, dtype=np.uint8).tobytes()
    s = matio.lz4_stream_compress(data)
    assert s[:8] == b"LZ4Block" and s[-21:] == b"LZ4Block" + bytes([0x16]) + bytes(12)
    token, clen, olen, check = struct.unpack_from("<BiiI", s, 8)
    assert token == 0x26 and olen == 65536 and clen < 400           # LZ4 method, 64 KiB blocks
    assert check == matio.xxh32(data[:65536], 0x9747B28C) & 0x0FFFFFFF
    methods, at = [], 0
    while at < len(s):
        token, clen, olen, _ = struct.unpack_from("<BiiI", s, at + 8)
        methods.append(token & 0xF0)
        at += 21 + clen
    assert methods == [0x20, 0x20, 0x10, 0x10]                       # zeros, zeros + random, random tail, end mark
    assert matio.lz4_stream_decompress(s) == data
    bad = bytearray(s)
    bad[30] ^= 1
    with pytest.raises(ValueError):
        matio.lz4_stream_decompress(bytes(bad))


@pytest.mark.parametrize("ext", ["", ".gz", ".lz4"])
@pytest.mark.parametrize("dtype,code", [(np.int32, 110), (np.int64, 120), (np.float32, 130), (np.float64, 140)])
def test_matrix_files_round_trip(tmp_path, ext, dtype, code):
    from bidmach_b200 import matio
    rng = np.random.default_rng(3)
    a = (rng.standard_normal((7, 1234)) * 100).astype(dtype)
    f = str(tmp_path / ("m.mat" + ext))
    matio.saveMat(f, a)
    b = matio.loadMat(f)
    assert b.dtype == dtype and np.array_equal(a, b) and matio.peekShape(f) == (7, 1234)
    raw = open(f, "rb").read()
    if ext == ".gz":
        raw = gzip.decompress(raw)
    if ext == ".lz4":
        raw = matio.lz4_stream_decompress(raw)
    # header and column-major payload exactly as the reference's C writers lay them out
    # (src/main/C/newparse/utils.cpp:350-362, 484-509)
    assert struct.unpack_from("<iiii", raw, 0) == (code, 7, 1234, 0)
    assert raw[16:] == np.asfortranarray(a).tobytes(order="F")


def test_vector_file_as_the_reference_c_writer_emits_it(tmp_path):
    """writeIntVec (utils.cpp:350-362): fmt 110, nrows = n, ncols = 1, nnz = n, then the ints."""
    from bidmach_b200 import matio
    v = np.array([5, 7, 11, 13], np.int32)
    ref_bytes = struct.pack("<iiii", 110, 4, 1, 4) + v.tobytes()
    f = str(tmp_path / "v.imat")
    matio.saveMat(f, v)
    assert open(f, "rb").read() == ref_bytes
    g = str(tmp_path / "w.imat")
    open(g, "wb").write(ref_bytes)
    assert np.array_equal(matio.loadMat(g).ravel(), v)


def test_token_files_are_the_minibatch_layout(tmp_path):
    from bidmach_b200 import matio
    toks = np.stack([np.arange(10, dtype=np.int32) * 3, np.arange(10, dtype=np.int32) // 4], axis=1)
    f = str(tmp_path / "train00000.imat.lz4")
    matio.saveTokens(f, toks)
    m = matio.loadMat(f)
    assert m.shape == (2, 10) and np.array_equal(m[0], toks[:, 0]) and np.array_equal(m[1], toks[:, 1])
    assert np.array_equal(matio.loadTokens(f), toks)


def _write_corpus(tmp_path, sizes, ext=".imat.lz4"):
    from bidmach_b200 import matio
    pat = str(tmp_path / ("train%05d" + ext))
    at = 0
    for i, n in enumerate(sizes):
        t = np.stack([np.arange(at, at + n, dtype=np.int32), np.full(n, i, np.int32)], axis=1)
        matio.saveTokens(pat % i, t)
        at += n
    return pat, at


@pytest.mark.parametrize("lookahead", [0, 2])
def test_filesource_stitches_minibatches_across_files(tmp_path, lookahead):
    """FileSource.next (FileSource.scala:185-223): a minibatch that reaches the end of a
    file is completed from the head of the next; only the last one is short."""
    from bidmach_b200.filesource import FileSource, FileSourceOpts, simpleEnum
    pat, total = _write_corpus(tmp_path, [250, 100, 330])
    ds = FileSource(FileSourceOpts(fnames=simpleEnum(pat), batchSize=100, lookahead=lookahead))
    got, sizes = [], []
    while ds.hasNext():
        b = ds.next()[0]
        sizes.append(b.shape[0])
        got.append(b[:, 0])
        assert 0.0 <= ds.progress() <= 1.0
    assert np.array_equal(np.concatenate(got), np.arange(total))
    assert sizes == [100, 100, 100, 100, 100, 100, 80]
    ds.reset()
    assert np.array_equal(ds.next()[0][:, 0], np.arange(100))
    ds.close()


def test_filesource_short_next_file_gives_the_reference_cut(tmp_path):
    """A minibatch spans at most two files: 30 tokens left + a 20-token file = 50; the
    walk then stands at the end of the short file, takes the next minibatch wholly from
    the file after it, and ends with the empty remainder of that one."""
    from bidmach_b200.filesource import FileSource, FileSourceOpts, count_minibatches, simpleEnum
    pat, total = _write_corpus(tmp_path, [130, 20, 100], ext=".imat")
    ds = FileSource(FileSourceOpts(fnames=simpleEnum(pat), batchSize=100, lookahead=1))
    sizes = []
    while ds.hasNext():
        sizes.append(ds.next()[0].shape[0])
    ds.close()
    assert sizes == [100, 50, 100, 0] and count_minibatches([130, 20, 100], 100) == 4


def test_filesource_deals_minibatches_to_replicas(tmp_path):
    from bidmach_b200.filesource import FileSource, FileSourceOpts, simpleEnum
    pat, total = _write_corpus(tmp_path, [250, 250, 250], ext=".imat.gz")     # 8 minibatches of 100 (last 50)
    seen = []
    for rank in range(3):
        ds = FileSource(FileSourceOpts(fnames=simpleEnum(pat), batchSize=100), offset=rank, stride=3)
        mine = []
        while ds.hasNext():
            mine.append(int(ds.next()[0][0, 0]) // 100)
        ds.close()
        seen.append(mine)
    assert seen == [[0, 3], [1, 4], [2, 5]]          # 8 minibatches -> 2 full rounds of 3


def test_filesource_random_order_keeps_the_last_file_last(tmp_path):
    from bidmach_b200.filesource import FileSource, FileSourceOpts, simpleEnum
    pat, total = _write_corpus(tmp_path, [100] * 6, ext=".imat")
    ds = FileSource(FileSourceOpts(fnames=simpleEnum(pat), batchSize=100, order=1, seed=3))
    order = []
    while ds.hasNext():
        order.append(int(ds.next()[0][0, 1]))
    ds.close()
    assert sorted(order) == list(range(6)) and order[-1] == 5 and order != list(range(6))


def test_filesource_without_files_raises(tmp_path):
    from bidmach_b200.filesource import FileSource, FileSourceOpts, simpleEnum
    with pytest.raises(RuntimeError):
        FileSource(FileSourceOpts(fnames=simpleEnum(str(tmp_path / "none%05d.imat"))))


def test_lz4_stream_reader_against_a_file_bidmat_wrote():
    """Golden vector: the tail (last data block + end mark) of the one matrix file in the
    BIDMach checkout that BIDMat wrote through lz4-java, with the header fields of all its
    blocks (tests/golden/make_lz4_golden.py).  Pins the container: magic, token, the two
    lengths, the 28-bit XXH32 checksum with lz4-java's seed, the end mark."""
    import json
    import os

    from bidmach_b200 import matio
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    meta = json.load(open(os.path.join(here, "lz4block_meta.json")))
    tail = open(os.path.join(here, "lz4block_tail.bin"), "rb").read()
    last, end = meta["blocks"][-2], meta["blocks"][-1]
    assert tail[:8] == b"LZ4Block" and struct.unpack_from("<BiiI", tail, 8) == (
        last["token"], last["compressed"], last["original"], last["checksum"])
    assert last["token"] == 0x16 and end == {"offset": end["offset"], "token": 0x16, "compressed": 0,
                                             "original": 0, "checksum": 0}
    chunk = matio.lz4_stream_decompress(tail)                 # verifies the stored checksum
    assert len(chunk) == last["original"]
    assert matio.xxh32(chunk, 0x9747B28C) & 0x0FFFFFFF == last["checksum"]
    # this build's writer frames the same bytes identically (the block is incompressible: raw)
    assert matio.lz4_stream_compress(chunk) == tail
    from oracle.build import REF_ROOT
    src = os.path.join(REF_ROOT, meta["source"])
    if os.path.exists(src):                                  # the whole file, where the checkout is at hand
        payload = matio.lz4_stream_decompress(open(src, "rb").read())
        assert len(payload) == meta["payload_bytes"] and matio.xxh32(payload, 0) == meta["payload_xxh32_seed0"]
        assert list(struct.unpack_from("<6i", payload, 0)) == meta["matrix_header_ints"]


def test_learner_constructors_take_a_file_pattern(tmp_path):
    """Word2Vec.learner(fn1) / learnPar(fn1) (Word2Vec.scala:1240-1254, 1315): a file-name
    pattern selects a FileSource; replica r of n gets minibatches r, r + n, ..."""
    from bidmach_b200.filesource import FileSource
    from bidmach_b200.learner import MatSource
    from bidmach_b200.word2vec import Word2Vec
    pat, total = _write_corpus(tmp_path, [100, 100], ext=".imat.gz")
    src = Word2Vec._source(pat, 50, 1, 2)
    assert isinstance(src, FileSource)
    got = []
    while src.hasNext():
        got.append(int(src.next()[0][0, 0]))
    src.close()
    assert got == [50, 150]
    assert isinstance(Word2Vec._source(np.zeros((10, 2), np.int32), 5, 0, 1), MatSource)
