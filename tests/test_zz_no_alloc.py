"""word2vecEvalNegNoAlloc, the scoring entry point for callers that may not
allocate device memory (its scratch is an array compiled into the library),
checked through the C-ABI against the regular word2vecEvalNeg and against the
CPU oracle: same inputs, same score within the kernels' 1e-5 relative bar, on
two calls in a row (the second call finds the scratch array as the first one
left it).  This file is collected last so that a failure here cannot hide any
other test."""
import numpy as np
import pytest
import torch

from helpers import random_model, random_neg

pytestmark = pytest.mark.gpu
TOL = 1e-5


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.mark.parametrize("nwa,nwb,dim,ncols", [(5, 5, 300, 3001), (10, 5, 100, 700), (5, 10, 64, 513),
                                               (5, 1, 37, 255)])
def test_no_alloc_score_matches_regular_entry_point_twice(oracle, nwa, nwb, dim, ncols):
    from bidmach_b200 import CUMACH
    from bidmach_b200.cumach import word2vecEvalNegNoAlloc
    vocab = 2000
    for call in range(2):
        A, B = random_model(vocab, dim, 10 * call + dim, scale=2.0 / np.sqrt(dim))
        WA, WB = random_neg(ncols + call * 300, vocab, nwa, nwb, call + 1)
        n = WA.shape[0]
        dA, dB, dWA, dWB = dev(A), dev(B), dev(WA), dev(WB)
        want = torch.zeros(1, device="cuda")
        got = torch.zeros(1, device="cuda")
        assert CUMACH.word2vecEvalNeg(dim, n, nwa, nwb, dWA, dWB, dA, dB, want) == 0
        assert word2vecEvalNegNoAlloc(dim, n, nwa, nwb, dWA, dWB, dA, dB, got) == 0
        assert want.item() < 0
        assert abs(got.item() - want.item()) <= TOL * abs(want.item())
        cpu = oracle.word2vecEvalNeg(dim, n, nwa, nwb, WA, WB, A, B, 4)
        assert abs(got.item() - cpu) <= TOL * abs(cpu)


def test_no_alloc_near_its_column_limit_matches_the_oracle(oracle):
    """2,097,000 columns: 8192 blocks, every partial-sum slot of the built-in array in use."""
    from bidmach_b200.cumach import word2vecEvalNegNoAlloc
    vocab, dim, ncols = 5000, 16, 2_097_000
    for call in range(2):
        A, B = random_model(vocab, dim, 40 + call, scale=0.5)
        WA, WB = random_neg(ncols, vocab, 5, 5, 50 + call)
        got = torch.zeros(1, device="cuda")
        assert word2vecEvalNegNoAlloc(dim, ncols, 5, 5, dev(WA), dev(WB), dev(A), dev(B), got) == 0
        cpu = oracle.word2vecEvalNeg(dim, ncols, 5, 5, WA, WB, A, B, 8)
        assert abs(got.item() - cpu) <= TOL * abs(cpu)


def test_masked_ids_score_as_zero_rows_in_every_eval_neg_path(oracle):
    """An id of -1 (a word the caller masked out) counts as a zero row: each of its pairs adds
    log(1/2).  Same answer from word2vecEvalNeg (staged kernel, dim 300; generic kernel, dim 37),
    from word2vecEvalNegNoAlloc, and from the CPU oracle run with the masked ids pointed at an
    appended row of zeros."""
    from bidmach_b200 import CUMACH
    from bidmach_b200.cumach import word2vecEvalNegNoAlloc
    vocab, ncols = 900, 700
    for dim in (300, 37):
        A, B = random_model(vocab, dim, dim, scale=2.0 / np.sqrt(dim))
        WA, WB = random_neg(ncols, vocab, 5, 5, dim + 1)
        rng = np.random.default_rng(dim)
        WA[rng.random(WA.shape) < 0.1] = -1
        WB[rng.random(WB.shape) < 0.1] = -1
        Az, Bz = np.vstack([A, np.zeros((1, dim), np.float32)]), np.vstack([B, np.zeros((1, dim), np.float32)])
        cpu = oracle.word2vecEvalNeg(dim, ncols, 5, 5, np.where(WA < 0, vocab, WA), np.where(WB < 0, vocab, WB),
                                     Az, Bz, 2)
        dA, dB, dWA, dWB = dev(A), dev(B), dev(WA), dev(WB)
        a, b = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
        assert CUMACH.word2vecEvalNeg(dim, ncols, 5, 5, dWA, dWB, dA, dB, a) == 0
        assert word2vecEvalNegNoAlloc(dim, ncols, 5, 5, dWA, dWB, dA, dB, b) == 0
        assert abs(a.item() - cpu) <= TOL * abs(cpu) and abs(b.item() - cpu) <= TOL * abs(cpu)


def test_no_alloc_accumulates_and_handles_empty_input():
    from bidmach_b200.cumach import word2vecEvalNegNoAlloc
    A, B = random_model(100, 100, 1, scale=0.2)
    WA, WB = random_neg(50, 100, 5, 5, 2)
    dA, dB, dWA, dWB = dev(A), dev(B), dev(WA), dev(WB)
    ret = torch.zeros(1, device="cuda")
    assert word2vecEvalNegNoAlloc(100, 50, 5, 5, dWA, dWB, dA, dB, ret) == 0
    once = ret.item()
    assert word2vecEvalNegNoAlloc(100, 50, 5, 5, dWA, dWB, dA, dB, ret) == 0   # adds, like the regular one
    assert abs(ret.item() - 2 * once) <= 2 * TOL * abs(once)
    assert word2vecEvalNegNoAlloc(100, 0, 5, 5, dWA, dWB, dA, dB, ret) == 0
    assert abs(ret.item() - 2 * once) <= 2 * TOL * abs(once)


def test_no_alloc_refuses_what_its_scratch_cannot_hold(capfd):
    from bidmach_b200.cumach import word2vecEvalNegNoAlloc
    z = torch.zeros(16, dtype=torch.int32, device="cuda")
    m = torch.zeros(4, 100, device="cuda")
    r = torch.zeros(1, device="cuda")
    assert word2vecEvalNegNoAlloc(100, 2_097_153, 5, 5, z, z, m, m, r) == 1    # beyond the column limit
    assert word2vecEvalNegNoAlloc(100, 10, 4, 4, z, z, m, m, r) == 1           # unsupported shape
    assert r.item() == 0.0
