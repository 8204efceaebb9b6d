"""Google word2vec file format as the reference writes it
(networks/Word2Vec.scala:1332-1394): header, big-endian binary floats, Java %g text."""
import numpy as np
import pytest

from bidmach_b200.modelio import java_g, readGoogleW2V, saveGoogleW2V


def test_java_percent_g():
    # java.util.Formatter %g: 6 significant digits, no trailing-zero stripping
    assert java_g(0.0) == "0.00000"
    assert java_g(1.0) == "1.00000"
    assert java_g(0.5) == "0.500000"
    assert java_g(-0.00123456789) == "-0.00123457"
    assert java_g(123456.7) == "123457"
    assert java_g(1234567.0) == "1.23457e+06"
    assert java_g(0.0001) == "0.000100000"
    assert java_g(0.00001234) == "1.23400e-05"
    assert java_g(99999.96) == "100000"
    assert java_g(999999.5) == "1.00000e+06"


def test_binary_layout_is_header_word_space_bigendian_floats_newline(tmp_path):
    mod = np.array([[1.0, -2.5], [0.15625, 3.0]], np.float32)
    f = tmp_path / "m.bin"
    assert saveGoogleW2V(["the", "of", "extra"], mod, f, binary=True) == 2
    raw = f.read_bytes()
    assert raw == (b"2 2\n" + b"the " + bytes.fromhex("3f800000" "c0200000") + b"\n" +
                   b"of " + bytes.fromhex("3e200000" "40400000") + b"\n")


def test_text_layout(tmp_path):
    mod = np.array([[1.0, -0.00123456789]], np.float32)
    f = tmp_path / "m.txt"
    saveGoogleW2V(["w", "x"], mod, f, binary=False)
    assert f.read_bytes() == b"1 2\nw 1.00000 -0.00123457 \n"


@pytest.mark.parametrize("binary", [True, False])
def test_round_trip_and_dictionary_filtering(tmp_path, binary, capsys):
    rng = np.random.default_rng(0)
    mod = ((rng.random((50, 7), dtype=np.float32) - 0.5) / 7).astype(np.float32)
    words = ["w%d" % i for i in range(60)]
    f = tmp_path / "m"
    assert saveGoogleW2V(words, mod, f, binary) == 50
    index = {w: i for i, w in enumerate(words)}
    back = readGoogleW2V(f, index, 50, binary)
    if binary:
        assert np.array_equal(back, mod)
    else:
        assert np.allclose(back, mod, rtol=1e-5, atol=0)
    # n smaller than the file: later words are skipped; unknown words are skipped
    part = readGoogleW2V(f, index, 10, binary)
    assert part.shape == (10, 7) and np.allclose(part, mod[:10], rtol=1e-5)
    del index["w3"]
    holed = readGoogleW2V(f, index, 50, binary)
    assert not holed[3].any() and np.allclose(holed[4], mod[4], rtol=1e-5)
    # dictionary shorter than the model: only that many words, with the reference's warning
    assert saveGoogleW2V(words[:20], mod, f, binary) == 20
    assert "dictionary is smaller" in capsys.readouterr().out


def test_accepts_torch_tensors(tmp_path):
    import torch
    mod = torch.arange(6, dtype=torch.float32).view(3, 2)
    f = tmp_path / "t.bin"
    saveGoogleW2V(["a", "b", "c", "d"], mod, f, binary=True)
    back = readGoogleW2V(f, {"a": 0, "b": 1, "c": 2}, 3, binary=True)
    assert np.array_equal(back, mod.numpy())


def test_checkpoint_directory_layout_and_round_trip(tmp_path):
    """Model.save (models/Model.scala:245-263): options.json + modelmat%02d.lz4, each a
    dim x vocab column-major float matrix."""
    import json
    import struct

    from bidmach_b200 import matio, modelio
    rng = np.random.default_rng(0)
    m0 = rng.standard_normal((50, 8)).astype(np.float32)      # [vocab, dim]
    m1 = rng.standard_normal((50, 8)).astype(np.float32)
    d = str(tmp_path / "ckpt") + "/"
    modelio.saveModel(d, {"dim": 8, "vocabSize": 50, "nskip": 5}, [m0, m1])
    assert sorted(p.name for p in (tmp_path / "ckpt").iterdir()) == ["modelmat00.lz4", "modelmat01.lz4",
                                                                    "options.json"]
    assert json.load(open(d + "options.json"))["vocabSize"] == 50
    raw = matio.lz4_stream_decompress(open(d + "modelmat00.lz4", "rb").read())
    assert struct.unpack_from("<iiii", raw, 0) == (130, 8, 50, 0)     # FMat, dim rows, vocab columns
    assert raw[16:] == m0.tobytes()                                    # word w = column w = 8 contiguous floats
    opts, mats = modelio.loadModel(d)
    assert opts["dim"] == 8 and len(mats) == 2
    assert np.array_equal(mats[0], m0) and np.array_equal(mats[1], m1)
