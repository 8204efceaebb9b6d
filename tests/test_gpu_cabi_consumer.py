"""The library used from a plain CUDA C++ program (no Python, no PyTorch in the
process): tests/cabi_consumer.cu is compiled against include/bidmach_b200.h,
linked with the shared library and run; its results are checked against the
CPU oracle."""
import os
import shutil
import subprocess

import numpy as np
import pytest

from helpers import conflict_free_neg, random_model, rel_err

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_c_program_links_and_matches_oracle(oracle, tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available to build the consumer")
    from bidmach_b200 import _lib
    libdir = os.path.dirname(_lib.LIB_PATH)
    exe = tmp_path / "cabi_consumer"
    subprocess.check_call([nvcc, "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "cabi_consumer.cu"), "-o", str(exe),
                           "-L", libdir, "-l:" + _lib.LIB_NAME, "-Xlinker", "-rpath", "-Xlinker", libdir])
    dim, vocab, ncols, nwa, nwb = 300, 4000, 390, 5, 5
    lrate, vexp = np.float32(0.02), np.float32(0.5)
    A, B = random_model(vocab, dim, 21, scale=0.5 / np.sqrt(dim))
    WA, WB = conflict_free_neg(ncols, vocab, nwa, nwb, 22)
    inp, out = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(inp, "wb") as f:
        f.write(np.array([dim, vocab, ncols, nwa, nwb], np.int32).tobytes())
        f.write(np.array([lrate, vexp], np.float32).tobytes())
        for x in (WA, WB, A, B):
            f.write(np.ascontiguousarray(x).tobytes())
    res = subprocess.run([str(exe), str(inp), str(out)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr + res.stdout
    assert "word2vec unsupport size combination 3 3" in res.stdout      # the reference's message
    lines = res.stdout.strip().splitlines()
    assert lines[-1].startswith("ok launches=")
    # the whole-minibatch calls: training on a minibatch raises its own score from 2*log(1/2)
    import re
    m = re.match(r"minibatch pairs=(\d+) score (-?[\d.]+) -> (-?[\d.]+)", lines[-2])
    assert m and int(m.group(1)) > 10000
    assert abs(float(m.group(2)) - 2 * np.log(0.5)) < 2e-3 and float(m.group(3)) > float(m.group(2)) + 0.05
    raw = np.fromfile(out, np.float32)
    scores, gA, gB = raw[:2], raw[2:2 + vocab * dim].reshape(vocab, dim), raw[2 + vocab * dim:].reshape(vocab, dim)
    want = oracle.word2vecEvalNeg(dim, ncols, nwa, nwb, WA, WB, A, B)
    assert abs(scores[0] - want) <= 1e-5 * abs(want) and abs(scores[1] - want) <= 1e-5 * abs(want)
    A_ref, B_ref = A.copy(), B.copy()
    oracle.word2vecNeg(dim, ncols, nwa, nwb, WA, WB, A_ref, B_ref, lrate, vexp, 1)
    assert rel_err(gA - A, A_ref - A) <= 1e-5 and rel_err(gB - B, B_ref - B) <= 1e-5
