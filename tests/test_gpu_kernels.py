"""Parity of the four CUDA kernels with the CPU oracle, called through the
C-ABI (the CUMACH entry points).  Updates are compared on conflict-free inputs
(where sequential and parallel execution agree) to 1e-5 of the largest change;
scores are compared on arbitrary inputs to 1e-5 relative."""
import numpy as np
import pytest
import torch

from helpers import (conflict_free_neg, conflict_free_pos, random_model, random_neg, random_pos,
                     rel_err)

pytestmark = pytest.mark.gpu

TOL = 1e-5  # relative, fp32 kernels vs the CPU reference


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.fixture(scope="module")
def cumach():
    from bidmach_b200 import CUMACH
    return CUMACH


def _pos_case(oracle, cumach, dim, vocab, ncols, skip, seed, lrate=0.05, vexp=0.5, drop=0.1):
    A, B = random_model(vocab, dim, seed, scale=0.5)
    W, LB, UB = conflict_free_pos(ncols, vocab, skip, seed, drop=drop)
    A_ref, B_ref = A.copy(), B.copy()
    oracle.word2vecPos(dim, ncols, skip, W, LB, UB, A_ref, B_ref, lrate, vexp, 1)
    dA, dB = dev(A), dev(B)
    err = cumach.word2vecPos(dim, ncols, skip, dev(W), dev(LB), dev(UB), dA, dB, lrate, vexp)
    assert err == 0
    gA, gB = dA.cpu().numpy(), dB.cpu().numpy()
    assert np.abs(A_ref - A).max() > 0
    assert rel_err(gA - A, A_ref - A) <= TOL
    assert rel_err(gB - B, B_ref - B) <= TOL
    untouched = np.setdiff1d(np.arange(vocab), W[W >= 0])
    assert np.array_equal(gA[untouched], A[untouched]) and np.array_equal(gB[untouched], B[untouched])


@pytest.mark.parametrize("dim", [100, 300, 64, 4, 512, 1280])
@pytest.mark.parametrize("skip", [5, 3, 2])
def test_pos_update_matches_oracle(oracle, cumach, dim, skip):
    _pos_case(oracle, cumach, dim, vocab=3000, ncols=2500, skip=skip, seed=dim + skip)


@pytest.mark.parametrize("dim", [100, 300, 512])
@pytest.mark.parametrize("drop", [0.0, 0.24, 0.26, 0.6])
def test_pos_update_dense_and_sparse_text(oracle, cumach, dim, drop):
    """Text with three quarters or more of its positions filled goes to the kernel that takes
    two centres at a time, sparser text to the one that takes one: both sides of the switch."""
    _pos_case(oracle, cumach, dim, vocab=6000, ncols=5001, skip=5, seed=int(dim + 100 * drop), drop=drop)


@pytest.mark.parametrize("dim", [37, 301, 1])
def test_pos_update_odd_dims_use_fallback(oracle, cumach, dim):
    _pos_case(oracle, cumach, dim, vocab=800, ncols=700, skip=5, seed=dim)


def test_pos_vexp_zero_and_large_ids(oracle, cumach):
    _pos_case(oracle, cumach, 100, vocab=200_000, ncols=3000, skip=5, seed=3, vexp=0.0)
    _pos_case(oracle, cumach, 100, vocab=200_000, ncols=3000, skip=5, seed=4, vexp=0.5)


def _neg_case(oracle, cumach, dim, vocab, ncols, nwa, nwb, seed, lrate=0.02, vexp=0.5):
    A, B = random_model(vocab, dim, seed, scale=0.5)
    WA, WB = conflict_free_neg(ncols, vocab, nwa, nwb, seed)
    A_ref, B_ref = A.copy(), B.copy()
    oracle.word2vecNeg(dim, ncols, nwa, nwb, WA, WB, A_ref, B_ref, lrate, vexp, 1)
    dA, dB = dev(A), dev(B)
    err = cumach.word2vecNeg(dim, ncols, nwa, nwb, dev(WA), dev(WB), dA, dB, lrate, vexp)
    assert err == 0
    gA, gB = dA.cpu().numpy(), dB.cpu().numpy()
    assert rel_err(gA - A, A_ref - A) <= TOL
    assert rel_err(gB - B, B_ref - B) <= TOL


@pytest.mark.parametrize("nwa,nwb", [(5, 1), (5, 5), (10, 5), (5, 10)])
@pytest.mark.parametrize("dim", [100, 300, 64, 256, 512])
def test_neg_update_matches_oracle(oracle, cumach, nwa, nwb, dim):
    _neg_case(oracle, cumach, dim, vocab=4000, ncols=390, nwa=nwa, nwb=nwb, seed=dim + nwa + nwb)


@pytest.mark.parametrize("dim", [37, 640, 1284])
def test_neg_update_fallback_dims(oracle, cumach, dim):
    _neg_case(oracle, cumach, dim, vocab=1000, ncols=90, nwa=5, nwb=5, seed=dim)


def test_neg_single_column_and_duplicates_inside_a_column(oracle, cumach):
    """One column whose A-words repeat: sequential and parallel still agree,
    because a column is one unit of work and A rows are written once at its end."""
    dim, vocab = 100, 50
    A, B = random_model(vocab, dim, 1, scale=0.5)
    WA = np.array([[3, 3, 7, 9, 3]], np.int32)
    WB = np.array([[1, 2, 4, 5, 6]], np.int32)
    A_ref, B_ref = A.copy(), B.copy()
    oracle.word2vecNeg(dim, 1, 5, 5, WA, WB, A_ref, B_ref, 0.02, 0.5, 1)
    dA, dB = dev(A), dev(B)
    assert cumach.word2vecNeg(dim, 1, 5, 5, dev(WA), dev(WB), dA, dB, 0.02, 0.5) == 0
    assert rel_err(dA.cpu().numpy() - A, A_ref - A) <= TOL
    assert rel_err(dB.cpu().numpy() - B, B_ref - B) <= TOL


def test_negfilt_masks_words_at_or_above_nwords(oracle, cumach):
    dim, vocab, ncols, nwords = 100, 600, 50, 300
    A, B = random_model(vocab, dim, 2, scale=0.5)
    WA, WB = conflict_free_neg(ncols, vocab, 5, 5, 2)
    A_ref, B_ref = A.copy(), B.copy()
    oracle.word2vecNegFilt(dim, ncols, nwords, 5, 5, WA, WB, A_ref, B_ref, 0.02, 0.5)
    dA, dB = dev(A), dev(B)
    assert cumach.word2vecNegFilt(dim, ncols, nwords, 5, 5, dev(WA), dev(WB), dA, dB, 0.02, 0.5) == 0
    gA, gB = dA.cpu().numpy(), dB.cpu().numpy()
    assert np.array_equal(gA[nwords:], A[nwords:]) and np.array_equal(gB[nwords:], B[nwords:])
    assert rel_err(gA - A, A_ref - A) <= 2e-5 and rel_err(gB - B, B_ref - B) <= 2e-5


@pytest.mark.parametrize("dim,skip", [(100, 5), (300, 5), (300, 3), (64, 2), (37, 5), (1280, 5)])
def test_eval_pos_matches_oracle(oracle, cumach, dim, skip):
    vocab, ncols = 2000, 5000
    A, B = random_model(vocab, dim, dim, scale=2.0 / np.sqrt(dim))
    W, LB, UB = random_pos(ncols, vocab, skip, dim + 1)
    want = oracle.word2vecEvalPos(dim, ncols, skip, W, LB, UB, A, B, 4)
    ret = torch.zeros(1, device="cuda")
    assert cumach.word2vecEvalPos(dim, ncols, skip, dev(W), dev(LB), dev(UB), dev(A), dev(B), ret) == 0
    assert abs(ret.item() - want) <= TOL * abs(want)
    # accumulates into the caller's value (the caller clears it)
    assert cumach.word2vecEvalPos(dim, ncols, skip, dev(W), dev(LB), dev(UB), dev(A), dev(B), ret) == 0
    assert abs(ret.item() - 2 * want) <= 2 * TOL * abs(want)


@pytest.mark.parametrize("nwa,nwb", [(5, 1), (5, 5), (10, 5), (5, 10)])
@pytest.mark.parametrize("dim", [100, 300, 37, 640])
def test_eval_neg_matches_oracle(oracle, cumach, nwa, nwb, dim):
    vocab, ncols = 2000, 1500
    A, B = random_model(vocab, dim, dim, scale=2.0 / np.sqrt(dim))
    WA, WB = random_neg(ncols, vocab, nwa, nwb, dim + 2)
    want = oracle.word2vecEvalNeg(dim, ncols, nwa, nwb, WA, WB, A, B, 4)
    ret = torch.zeros(1, device="cuda")
    assert cumach.word2vecEvalNeg(dim, ncols, nwa, nwb, dev(WA), dev(WB), dev(A), dev(B), ret) == 0
    assert abs(ret.item() - want) <= TOL * abs(want)


def test_eval_saturated_scores_hit_the_clamp(oracle, cumach):
    """Dots beyond +-16 give sigmoid exactly 1 / 0 and log(1e-20) for the clamped side."""
    dim, vocab = 100, 20
    A = np.full((vocab, dim), 1.0, np.float32)
    B = np.full((vocab, dim), -1.0, np.float32)  # every dot is -100
    W = np.arange(10, dtype=np.int32)
    LB, UB = np.full(10, -1, np.int32), np.full(10, 1, np.int32)
    LB[0], UB[-1] = 0, 0
    want = oracle.word2vecEvalPos(dim, 10, 5, W, LB, UB, A, B)
    ret = torch.zeros(1, device="cuda")
    assert cumach.word2vecEvalPos(dim, 10, 5, dev(W), dev(LB), dev(UB), dev(A), dev(B), ret) == 0
    assert abs(want - 18 * np.log(1e-20)) < 1e-6 and abs(ret.item() - want) <= TOL * abs(want)


def test_unsupported_shapes_return_one_like_the_reference(cumach, capfd):
    z = torch.zeros(16, dtype=torch.int32, device="cuda")
    m = torch.zeros(4, 100, device="cuda")
    big = torch.zeros(2, 1284, device="cuda")
    r = torch.zeros(1, device="cuda")
    assert cumach.word2vecPos(100, 4, 4, z, z, z, m, m, 0.1, 0.5) == 1
    assert cumach.word2vecPos(1284, 1, 5, z, z, z, big, big, 0.1, 0.5) == 1
    assert cumach.word2vecNeg(100, 1, 4, 4, z, z, m, m, 0.1, 0.5) == 1
    assert cumach.word2vecNegFilt(100, 1, 4, 7, 3, z, z, m, m, 0.1, 0.5) == 1
    assert cumach.word2vecEvalPos(100, 4, 7, z, z, z, m, m, r) == 1
    assert cumach.word2vecEvalNeg(100, 1, 15, 10, z, z, m, m, r) == 1


def test_empty_and_all_masked_inputs_change_nothing(cumach):
    A, B = random_model(50, 100, 0)
    dA, dB = dev(A), dev(B)
    W = dev(np.full(64, -1, np.int32))
    LB, UB = dev(np.full(64, -5, np.int32)), dev(np.full(64, 5, np.int32))
    assert cumach.word2vecPos(100, 64, 5, W, LB, UB, dA, dB, 0.1, 0.5) == 0
    assert cumach.word2vecPos(100, 0, 5, W, LB, UB, dA, dB, 0.1, 0.5) == 0
    assert cumach.word2vecNeg(100, 0, 5, 5, W, W, dA, dB, 0.1, 0.5) == 0
    ret = torch.zeros(1, device="cuda")
    assert cumach.word2vecEvalPos(100, 64, 5, W, LB, UB, dA, dB, ret) == 0
    assert cumach.word2vecEvalNeg(100, 0, 5, 5, W, W, dA, dB, ret) == 0
    assert ret.item() == 0.0
    assert np.array_equal(dA.cpu().numpy(), A) and np.array_equal(dB.cpu().numpy(), B)


def test_zero_learning_rate_is_the_identity_on_conflicting_input(cumach):
    A, B = random_model(300, 300, 1)
    dA, dB = dev(A), dev(B)
    W, LB, UB = random_pos(20000, 300, 5, 2)
    WA, WB = random_neg(4000, 300, 5, 5, 3)
    assert cumach.word2vecPos(300, 20000, 5, dev(W), dev(LB), dev(UB), dA, dB, 0.0, 0.5) == 0
    assert cumach.word2vecNeg(300, 4000, 5, 5, dev(WA), dev(WB), dA, dB, 0.0, 0.5) == 0
    assert np.array_equal(dA.cpu().numpy(), A) and np.array_equal(dB.cpu().numpy(), B)


def test_conflicting_updates_lose_nothing(oracle, cumach):
    """Hot rows: every row is updated by about 25 columns at once.  With a small
    learning rate the gradients barely depend on the order in which concurrent
    units read the rows (sequential and fully parallel evaluation differ by
    about 1e-3 here), so the atomically accumulated result must match the
    sequential one closely; a single lost row update would leave a gap of about
    1/25 = 4e-2."""
    dim, vocab, ncols = 100, 40, 200
    A, B = random_model(vocab, dim, 5, scale=0.01)
    WA, WB = random_neg(ncols, vocab, 5, 5, 6)
    lr = 2e-5
    A_ref, B_ref = A.copy(), B.copy()
    oracle.word2vecNeg(dim, ncols, 5, 5, WA, WB, A_ref, B_ref, lr, 0.0, 1)
    dA, dB = dev(A), dev(B)
    assert cumach.word2vecNeg(dim, ncols, 5, 5, dev(WA), dev(WB), dA, dB, lr, 0.0) == 0
    assert rel_err(dA.cpu().numpy() - A, A_ref - A) <= 5e-3
    assert rel_err(dB.cpu().numpy() - B, B_ref - B) <= 5e-3
    # the same for positive pairs: every position is a centre with a full window
    W, LB, UB = random_pos(1000, vocab, 5, 7, drop=0.0, doc_len=1000)
    A_ref, B_ref = A.copy(), B.copy()
    oracle.word2vecPos(dim, 1000, 5, W, LB, UB, A_ref, B_ref, lr, 0.0, 1)
    dA, dB = dev(A), dev(B)
    assert cumach.word2vecPos(dim, 1000, 5, dev(W), dev(LB), dev(UB), dA, dB, lr, 0.0) == 0
    assert rel_err(dA.cpu().numpy() - A, A_ref - A) <= 1e-2
    assert rel_err(dB.cpu().numpy() - B, B_ref - B) <= 1e-2


def test_golden_fixtures_on_gpu_conflict_free_prefix(oracle, cumach):
    """The committed fixtures hold general (conflicting) inputs, so only their
    scores are compared on the GPU: eval of the reference's post-update model."""
    import glob
    import os
    for f in sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "kernels_*.npz"))):
        g = np.load(f)
        dim, skip = int(g["dim"]), int(g["skip"])
        if skip not in (2, 3, 5):
            continue
        A, B = g["A_neg"], g["B_neg"]
        want = oracle.word2vecEvalPos(dim, len(g["W"]), skip, g["W"], g["LB"], g["UB"], A, B)
        ret = torch.zeros(1, device="cuda")
        assert cumach.word2vecEvalPos(dim, len(g["W"]), skip, dev(g["W"]), dev(g["LB"]), dev(g["UB"]),
                                      dev(A), dev(B), ret) == 0
        assert abs(ret.item() - want) <= TOL * abs(want)


def test_apply_average_adds_the_difference():
    """w2v_apply_average: theta += avg - base (second half of the overlapped model average)."""
    from bidmach_b200 import _lib
    lib = _lib.load()
    torch.manual_seed(0)
    theta = torch.randn(1000, 300, device="cuda")
    base = torch.randn_like(theta)
    avg = torch.randn_like(theta)
    want = theta + (avg - base)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.w2v_apply_average(theta.data_ptr(), base.data_ptr(), avg.data_ptr(), theta.numel(), stream) == 0
    torch.cuda.synchronize()
    assert torch.allclose(theta, want, rtol=0, atol=1e-6)
    assert lib.w2v_apply_average(theta.data_ptr(), base.data_ptr(), avg.data_ptr(), 7, stream) == 1


@pytest.mark.parametrize("dim,drop", [(300, 0.0), (300, 0.3), (100, 0.15), (64, 0.0)])
def test_pos_adjacent_centres_match_a_jacobi_reference(dim, drop):
    """Every position a centre with its own window, all words distinct: every gradient is
    then a function of the initial rows only (an A row is written by its own centre after it
    was read; a B row when the window has passed), so the result must equal the sums below up
    to fp32 order.  This is the input on which neighbouring centres share their context rows
    (the two-centres-at-a-time path).  Positions near the seams between the four warps'
    stretches are left out of the comparison: there a row may be read after the neighbouring
    warp has already added its delta."""
    from bidmach_b200 import CUMACH
    n, V, skip, lr, vexp = 400, 1000, 5, 0.05, 0.5
    rng = np.random.default_rng(int(dim + 100 * drop))
    W = rng.permutation(V)[:n].astype(np.int32)
    W[rng.random(n) < drop] = -1
    ub = rng.integers(1, skip + 1, n).astype(np.int32)
    LB, UB = (-ub).astype(np.int32), ub.copy()
    A0, B0 = random_model(V, dim, 7, scale=0.5)
    dA, dB = np.zeros((V, dim)), np.zeros((V, dim))
    A64, B64 = A0.astype(np.float64), B0.astype(np.float64)
    for t in range(n):
        if W[t] < 0:
            continue
        for j in range(LB[t], UB[t] + 1):
            u = t + j
            if j == 0 or u < 0 or u >= n or W[u] < 0:
                continue
            d = float(np.float32(A64[W[t]] @ B64[W[u]]))
            g = lr * (1.0 - (1.0 if d > 16 else 0.0 if d < -16 else np.exp(d) / (1 + np.exp(d))))
            dA[W[t]] += (1.0 + W[t]) ** vexp * g * B64[W[u]]
            dB[W[u]] += (1.0 + W[u]) ** vexp * g * A64[W[t]]
    gA, gB = dev(A0), dev(B0)
    assert CUMACH.word2vecPos(dim, n, skip, dev(W), dev(LB), dev(UB), gA, gB, lr, vexp) == 0
    gotA, gotB = gA.cpu().numpy().astype(np.float64) - A64, gB.cpu().numpy().astype(np.float64) - B64
    seams = [100, 200, 300]                       # one block of four warps: stretches of 100 positions
    inner = np.array([t for t in range(n) if W[t] >= 0 and all(abs(t - s) > 2 * skip + 2 for s in seams)])
    assert len(inner) > 150
    rows = W[inner]
    assert rel_err(gotA[rows], dA[rows]) <= 1e-5
    assert rel_err(gotB[rows], dB[rows]) <= 1e-5
    # nothing outside the minibatch's words moved
    untouched = np.setdiff1d(np.arange(V), W[W >= 0])
    assert not gotA[untouched].any() and not gotB[untouched].any()
