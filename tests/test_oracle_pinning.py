"""Pins the C restatement (oracle/w2v_oracle.c) to the reference's own CPU
kernels: bit for bit against the compiled reference where it was built, and
against the committed fixtures that were generated from it."""
import glob
import os

import numpy as np
import pytest

from helpers import random_model, random_neg, random_pos

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _cases():
    return [(100, 400, 5, 300, 1), (300, 500, 5, 200, 2), (64, 50, 3, 257, 3), (37, 80, 2, 64, 4)]


@pytest.mark.parametrize("dim,vocab,skip,ncols,seed", _cases())
def test_port_equals_compiled_reference_pos(oracle, dim, vocab, skip, ncols, seed):
    if not oracle.have_reference():
        pytest.skip("compiled reference not present on this machine")
    A, B = random_model(vocab, dim, seed, scale=0.5)
    W, LB, UB = random_pos(ncols, vocab, skip, seed)
    A1, B1, A2, B2 = A.copy(), B.copy(), A.copy(), B.copy()
    oracle.word2vecPos(dim, ncols, skip, W, LB, UB, A1, B1, 0.05, 0.5, 1, "port")
    oracle.word2vecPos(dim, ncols, skip, W, LB, UB, A2, B2, 0.05, 0.5, 1, "reference")
    assert np.array_equal(A1, A2) and np.array_equal(B1, B2)
    assert not np.array_equal(A1, A)


@pytest.mark.parametrize("nwa,nwb", [(5, 1), (5, 5), (10, 5), (5, 10)])
@pytest.mark.parametrize("dim", [100, 300])
def test_port_equals_compiled_reference_neg(oracle, nwa, nwb, dim):
    if not oracle.have_reference():
        pytest.skip("compiled reference not present on this machine")
    vocab, ncols = 300, 120
    A, B = random_model(vocab, dim, 7, scale=0.5)
    WA, WB = random_neg(ncols, vocab, nwa, nwb, 11)
    A1, B1, A2, B2 = A.copy(), B.copy(), A.copy(), B.copy()
    oracle.word2vecNeg(dim, ncols, nwa, nwb, WA, WB, A1, B1, 0.02, 0.5, 1, "port")
    oracle.word2vecNeg(dim, ncols, nwa, nwb, WA, WB, A2, B2, 0.02, 0.5, 1, "reference")
    assert np.array_equal(A1, A2) and np.array_equal(B1, B2)


def test_port_equals_golden_fixtures(oracle):
    files = sorted(glob.glob(os.path.join(GOLD, "kernels_*.npz")))
    assert files, "golden fixtures missing"
    for f in files:
        g = np.load(f)
        dim, skip = int(g["dim"]), int(g["skip"])
        A, B = g["A"].copy(), g["B"].copy()
        oracle.word2vecPos(dim, len(g["W"]), skip, g["W"], g["LB"], g["UB"], A, B, float(g["lrate"]),
                           float(g["vexp"]), 1, "port")
        assert np.array_equal(A, g["A_pos"]) and np.array_equal(B, g["B_pos"]), f
        nwa, nwb = g["WA"].shape[1], g["WB"].shape[1]
        oracle.word2vecNeg(dim, g["WA"].shape[0], nwa, nwb, g["WA"], g["WB"], A, B,
                           float(g["lrate"]) / nwa, float(g["vexp"]), 1, "port")
        assert np.array_equal(A, g["A_neg"]) and np.array_equal(B, g["B_neg"]), f


def _eval_numpy(dim, W, LB, UB, A, B):
    tot = 0.0
    for i in range(len(W)):
        if W[i] < 0:
            continue
        for j in range(LB[i], UB[i] + 1):
            if j == 0 or not (0 <= i + j < len(W)) or W[i + j] < 0:
                continue
            x = float(np.dot(A[W[i]].astype(np.float64), B[W[i + j]].astype(np.float64)))
            s = 1.0 if x > 16 else 0.0 if x < -16 else 1.0 / (1.0 + np.exp(-x))
            tot += np.log(max(s, 1e-20))
    return tot


def test_eval_port_matches_float64_restatement(oracle):
    dim, vocab, ncols, skip = 100, 200, 400, 5
    A, B = random_model(vocab, dim, 3, scale=0.3)
    W, LB, UB = random_pos(ncols, vocab, skip, 5)
    got = oracle.word2vecEvalPos(dim, ncols, skip, W, LB, UB, A, B)
    want = _eval_numpy(dim, W, LB, UB, A, B)
    assert abs(got - want) <= 1e-5 * abs(want)
    WA, WB = random_neg(60, vocab, 5, 5, 9)
    got = oracle.word2vecEvalNeg(dim, 60, 5, 5, WA, WB, A, B)
    want = 0.0
    for c in range(60):
        for k in range(5):
            for j in range(5):
                x = float(np.dot(A[WA[c, j]].astype(np.float64), B[WB[c, k]].astype(np.float64)))
                s = 1.0 if x > 16 else 0.0 if x < -16 else 1.0 / (1.0 + np.exp(-x))
                want += np.log(max(1.0 - s, 1e-20))
    assert abs(got - want) <= 1e-5 * abs(want)


def test_eval_reference_c_is_close_when_its_accumulator_starts_clean(oracle):
    """The reference's C eval adds onto an uninitialised local; in practice it is
    zero, and then its result must agree with the port except for the 1e-40 clamp."""
    if not oracle.have_reference():
        pytest.skip("compiled reference not present on this machine")
    import ctypes as C
    dim, vocab, ncols, skip = 100, 200, 300, 5
    A, B = random_model(vocab, dim, 3, scale=1.0)
    W, LB, UB = random_pos(ncols, vocab, skip, 5)
    ref = oracle.ref_lib().ref_word2vecEvalPos(
        dim, ncols, skip, W.ctypes.data_as(C.POINTER(C.c_int)), LB.ctypes.data_as(C.POINTER(C.c_int)),
        UB.ctypes.data_as(C.POINTER(C.c_int)), A.ctypes.data_as(C.POINTER(C.c_float)),
        B.ctypes.data_as(C.POINTER(C.c_float)), 1)
    got = oracle.word2vecEvalPos(dim, ncols, skip, W, LB, UB, A, B)
    if np.isfinite(ref) and abs(ref) < 1e12:
        assert abs(got - ref) <= 1e-9 * abs(got)


def test_bounds_against_python_restatement(oracle):
    rng = np.random.default_rng(0)
    n, vocab, nskip = 500, 1000, 5
    toks = np.empty((n, 2), np.int32)
    toks[:, 0] = rng.integers(0, vocab + 50, size=n)
    toks[:, 1] = np.cumsum(rng.random(n) < 0.08)
    u1 = rng.random(n, dtype=np.float32)
    u2 = rng.random(n, dtype=np.float32)
    salpha = oracle.salpha_of(1e-4, vocab)
    words, lb, ub = oracle.wordmats_bounds(toks, vocab, nskip, salpha, u1, u2)
    for i in range(n):
        wid = toks[i, 0]
        x = np.float32(np.float32(wid + 1) * salpha)
        keep = wid < vocab and u1[i] < np.float32(np.sqrt(x) + x)
        assert words[i] == (wid if keep else -1)
        ubr = min(nskip, int(np.float32(u2[i] * np.float32(nskip))) + 1)
        s = i
        while s > 0 and toks[s - 1, 1] == toks[i, 1]:
            s -= 1
        e = i
        while e < n - 1 and toks[e + 1, 1] == toks[i, 1]:
            e += 1
        assert lb[i] == max(-ubr, s - i) and ub[i] == min(ubr, e - i)
    ctx = oracle.ordered_contexts(words, lb, ub)
    want = [words[i + j] for i in range(n) if words[i] >= 0
            for j in range(lb[i], ub[i] + 1) if j != 0 and words[i + j] >= 0]
    assert ctx.tolist() == want


def test_shuffle_and_negative_ids(oracle):
    rng = np.random.default_rng(1)
    n = 1000
    ctx = np.arange(n, dtype=np.int32)
    pr = rng.random(n)
    want = ctx.copy()
    for i in range(n):
        pick = min(n - 1, i + int(np.floor(pr[i] * (n - i))))
        if pick > i:
            want[i], want[pick] = want[pick], want[i]
    import ctypes as C
    got = ctx.copy()
    oracle.port_lib().orc_shuffle(C.c_int64(n), got.ctypes.data_as(C.POINTER(C.c_int)),
                                  pr.ctypes.data_as(C.POINTER(C.c_double)))
    assert np.array_equal(got, want) and sorted(got.tolist()) == list(range(n))
    u = rng.random(5000, dtype=np.float32)
    ids = oracle.negative_ids(u, oracle.expt_of(0.75), 1_000_000)
    want = np.minimum(999_999, (1_000_000 * u.astype(np.float64) ** 4.0).astype(np.int64))
    assert np.array_equal(ids, want.astype(np.int32))
    assert oracle.negative_ids(np.array([0.99999994], np.float32), np.float32(4.0), 10)[0] == 9


@pytest.mark.parametrize("nslices,islice,nhead,do_head", [(4, 1, 20, 1), (3, 0, 0, 1), (2, 1, 50, 0), (4, 3, 37, 2),
                                                          (8, 5, 16, 1)])
def test_port_equals_compiled_reference_slices(oracle, nslices, islice, nhead, do_head):
    """word2vecPosSlice / word2vecNegSlice: the restatement against the reference's own C, bit for
    bit, on general (conflicting) input with words of every kind: head, this slice's, other slices'."""
    if not oracle.have_reference():
        pytest.skip("compiled reference not present on this machine")
    dim, vocab, ncols = 64, 400, 600
    rows = oracle.slice_rows(vocab, nslices, nhead)
    A, B = random_model(rows, dim, 3 + nslices, scale=0.5)
    W, LB, UB = random_pos(ncols, vocab, 5, 5 + islice)
    A1, B1, A2, B2 = A.copy(), B.copy(), A.copy(), B.copy()
    oracle.word2vecPosSlice(dim, ncols, 5, W, LB, UB, A1, B1, 0.05, 0.5, islice, nslices, nhead, do_head, 1, "port")
    oracle.word2vecPosSlice(dim, ncols, 5, W, LB, UB, A2, B2, 0.05, 0.5, islice, nslices, nhead, do_head, 1,
                            "reference")
    assert np.array_equal(A1, A2) and np.array_equal(B1, B2)
    assert not np.array_equal(A1, A)
    if do_head == 0:
        assert np.array_equal(A1[:nhead], A[:nhead]) and np.array_equal(B1[:nhead], B[:nhead])
    WA, WB = random_neg(150, vocab, 5, 5, 9 + islice)
    oracle.word2vecNegSlice(dim, 150, 5, 5, WA, WB, A1, B1, 0.02, 0.5, islice, nslices, nhead, do_head, 1, "port")
    oracle.word2vecNegSlice(dim, 150, 5, 5, WA, WB, A2, B2, 0.02, 0.5, islice, nslices, nhead, do_head, 1,
                            "reference")
    assert np.array_equal(A1, A2) and np.array_equal(B1, B2)


def test_one_slice_without_head_is_the_plain_kernel(oracle):
    """nslices = 1, nhead = 0: every id is this slice's own, rows are where they always were."""
    dim, vocab, ncols = 32, 200, 300
    A, B = random_model(vocab, dim, 1, scale=0.5)
    W, LB, UB = random_pos(ncols, vocab, 3, 2)
    A1, B1, A2, B2 = A.copy(), B.copy(), A.copy(), B.copy()
    oracle.word2vecPos(dim, ncols, 3, W, LB, UB, A1, B1, 0.05, 0.5, 1, "port")
    oracle.word2vecPosSlice(dim, ncols, 3, W, LB, UB, A2, B2, 0.05, 0.5, 0, 1, 0, 1, 1, "port")
    assert np.array_equal(A1, A2) and np.array_equal(B1, B2)
    e1 = oracle.word2vecEvalPos(dim, ncols, 3, W, LB, UB, A1, B1)
    e2 = oracle.word2vecEvalPosSlice(dim, ncols, 3, W, LB, UB, A1, B1, 0, 1, 0)
    assert e1 == e2
    WA, WB = random_neg(80, vocab, 5, 5, 4)
    assert oracle.word2vecEvalNeg(dim, 80, 5, 5, WA, WB, A1, B1) == \
        oracle.word2vecEvalNegSlice(dim, 80, 5, 5, WA, WB, A1, B1, 0, 1, 0)


def test_port_equals_golden_slice_fixtures(oracle):
    """slices_*.npz were written by the reference's own word2vecPosSlice / word2vecNegSlice: the
    restatement reproduces them bit for bit, with or without the compiled reference at hand."""
    files = sorted(glob.glob(os.path.join(GOLD, "slices_*.npz")))
    assert files, "golden slice fixtures missing"
    for f in files:
        g = np.load(f)
        dim, skip = int(g["dim"]), int(g["skip"])
        sl = (int(g["islice"]), int(g["nslices"]), int(g["nhead"]), int(g["do_head"]))
        A, B = g["A"].copy(), g["B"].copy()
        oracle.word2vecPosSlice(dim, len(g["W"]), skip, g["W"], g["LB"], g["UB"], A, B, float(g["lrate"]),
                                float(g["vexp"]), *sl, 1, "port")
        assert np.array_equal(A, g["A_pos"]) and np.array_equal(B, g["B_pos"]), f
        nwa, nwb = g["WA"].shape[1], g["WB"].shape[1]
        oracle.word2vecNegSlice(dim, g["WA"].shape[0], nwa, nwb, g["WA"], g["WB"], A, B,
                                float(g["lrate"]) / nwa, float(g["vexp"]), *sl, 1, "port")
        assert np.array_equal(A, g["A_neg"]) and np.array_equal(B, g["B_neg"]), f
        assert not np.array_equal(g["A_neg"], g["A"])
