"""Vocabulary slices on the GPU (word2vecPosSlice / word2vecNegSlice / word2vecEvalPosSlice /
word2vecEvalNegSlice and the sliced whole-minibatch calls) against the CPU oracle, which for the
update kernels is the restatement pinned bit for bit to the reference's own C
(tests/test_oracle_pinning.py)."""
import os

import numpy as np
import pytest
import torch

from helpers import conflict_free_neg, conflict_free_pos, elem_rel_err, random_model, random_neg, random_pos, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-5
THREADS = min(16, os.cpu_count() or 1)
SLICINGS = [(4, 1, 20, 1), (3, 0, 0, 1), (2, 1, 50, 0), (4, 3, 37, 2), (8, 5, 16, 1)]


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.mark.parametrize("nslices,islice,nhead,do_head", SLICINGS)
@pytest.mark.parametrize("dim", [100, 300])
def test_pos_slice_matches_oracle_on_conflict_free_input(oracle, nslices, islice, nhead, do_head, dim):
    from bidmach_b200 import CUMACHSlice
    vocab, ncols, skip = 4000, 3500, 5
    rows = oracle.slice_rows(vocab, nslices, nhead)
    A, B = random_model(rows, dim, nslices + dim, scale=0.5)
    W, LB, UB = conflict_free_pos(ncols, vocab, skip, islice + 1)
    A_ref, B_ref = A.copy(), B.copy()
    oracle.word2vecPosSlice(dim, ncols, skip, W, LB, UB, A_ref, B_ref, 0.05, 0.5, islice, nslices, nhead, do_head)
    dA, dB = dev(A), dev(B)
    assert CUMACHSlice.word2vecPosSlice(dim, ncols, skip, dev(W), dev(LB), dev(UB), dA, dB, 0.05, 0.5,
                                        islice, nslices, nhead, do_head) == 0
    gA, gB = dA.cpu().numpy(), dB.cpu().numpy()
    assert np.abs(A_ref - A).max() > 0
    assert rel_err(gA - A, A_ref - A) <= TOL and rel_err(gB - B, B_ref - B) <= TOL
    assert elem_rel_err(gA - A, A_ref - A) <= 1e-4 and elem_rel_err(gB - B, B_ref - B) <= 1e-4
    # rows the oracle left alone are bit for bit what they were (head rows when do_head is 0 among them)
    same = np.all(A_ref == A, axis=1)
    assert np.array_equal(gA[same], A[same])
    same = np.all(B_ref == B, axis=1)
    assert np.array_equal(gB[same], B[same])


@pytest.mark.parametrize("nslices,islice,nhead,do_head", SLICINGS)
@pytest.mark.parametrize("nwa,nwb,dim", [(5, 5, 300), (10, 5, 100), (5, 10, 64), (5, 1, 100)])
def test_neg_slice_matches_oracle_on_conflict_free_input(oracle, nslices, islice, nhead, do_head, nwa, nwb, dim):
    from bidmach_b200 import CUMACHSlice
    vocab, ncols = 6000, 590
    rows = oracle.slice_rows(vocab, nslices, nhead)
    A, B = random_model(rows, dim, nslices + dim, scale=0.5)
    WA, WB = conflict_free_neg(ncols, vocab, nwa, nwb, islice + 3)
    A_ref, B_ref = A.copy(), B.copy()
    oracle.word2vecNegSlice(dim, ncols, nwa, nwb, WA, WB, A_ref, B_ref, 0.02, 0.5, islice, nslices, nhead, do_head)
    dA, dB = dev(A), dev(B)
    assert CUMACHSlice.word2vecNegSlice(dim, ncols, nwa, nwb, dev(WA), dev(WB), dA, dB, 0.02, 0.5,
                                        islice, nslices, nhead, do_head) == 0
    gA, gB = dA.cpu().numpy(), dB.cpu().numpy()
    assert np.abs(A_ref - A).max() > 0
    assert rel_err(gA - A, A_ref - A) <= TOL and rel_err(gB - B, B_ref - B) <= TOL
    assert elem_rel_err(gA - A, A_ref - A) <= 1e-4 and elem_rel_err(gB - B, B_ref - B) <= 1e-4
    same = np.all(A_ref == A, axis=1)
    assert np.array_equal(gA[same], A[same])
    same = np.all(B_ref == B, axis=1)
    assert np.array_equal(gB[same], B[same])


@pytest.mark.parametrize("nslices,islice,nhead,do_head", SLICINGS)
def test_eval_slices_match_oracle_on_general_input(oracle, nslices, islice, nhead, do_head):
    from bidmach_b200 import CUMACHSlice
    dim, vocab, ncols = 300, 3000, 5000
    rows = oracle.slice_rows(vocab, nslices, nhead)
    A, B = random_model(rows, dim, 7, scale=2.0 / np.sqrt(dim))
    W, LB, UB = random_pos(ncols, vocab, 5, 8 + islice)
    want = oracle.word2vecEvalPosSlice(dim, ncols, 5, W, LB, UB, A, B, islice, nslices, nhead, 4)
    ret = torch.zeros(1, device="cuda")
    assert CUMACHSlice.word2vecEvalPosSlice(dim, ncols, 5, dev(W), dev(LB), dev(UB), dev(A), dev(B), ret,
                                            islice, nslices, nhead) == 0
    assert want < 0 and abs(ret.item() - want) <= TOL * abs(want)
    for nwa, nwb in ((5, 5), (10, 5)):
        WA, WB = random_neg(1500, vocab, nwa, nwb, 9 + islice)
        want = oracle.word2vecEvalNegSlice(dim, 1500, nwa, nwb, WA, WB, A, B, islice, nslices, nhead, 4)
        ret = torch.zeros(1, device="cuda")
        assert CUMACHSlice.word2vecEvalNegSlice(dim, 1500, nwa, nwb, dev(WA), dev(WB), dev(A), dev(B), ret,
                                                islice, nslices, nhead) == 0
        assert want < 0 and abs(ret.item() - want) <= TOL * abs(want)


def test_all_slices_together_cover_what_the_whole_model_sees(oracle):
    """Slices partition the tail: with do_head 2 every pair of two words that share a slice (or
    involve the head) is scored by exactly the slices that hold both, so on a text whose tail
    words all fall into one slice the slice's score equals the whole-vocabulary score."""
    from bidmach_b200 import CUMACH, CUMACHSlice
    dim, vocab, ncols, nslices, nhead = 100, 2000, 3000, 4, 100
    A, B = random_model(vocab, dim, 3, scale=0.3)
    rng = np.random.default_rng(4)
    ids = np.arange(vocab)
    usable = ids[(ids < nhead) | (ids % nslices == 2)]
    W = rng.choice(usable, ncols).astype(np.int32)
    LB, UB = np.full(ncols, -3, np.int32), np.full(ncols, 3, np.int32)
    LB[:3], UB[-3:] = 0, 0
    whole = torch.zeros(1, device="cuda")
    assert CUMACH.word2vecEvalPos(dim, ncols, 3, dev(W), dev(LB), dev(UB), dev(A), dev(B), whole) == 0
    part = torch.zeros(1, device="cuda")
    As, Bs = oracle.slice_of_model(A, 2, nslices, nhead), oracle.slice_of_model(B, 2, nslices, nhead)
    assert CUMACHSlice.word2vecEvalPosSlice(dim, ncols, 3, dev(W), dev(LB), dev(UB), dev(As), dev(Bs), part,
                                            2, nslices, nhead) == 0
    assert abs(part.item() - whole.item()) <= TOL * abs(whole.item())


def test_sliced_minibatch_calls_follow_the_slice_kernels(oracle):
    """Word2Vec with nSlices > 1: init sizes the matrices to the slice, dobatch / evalbatch work
    on the slice's pairs.  One minibatch with learning rate 0 changes nothing; with a rate the
    slice's held-out score moves, and rows of the head stay put when doHead is 0."""
    from bidmach_b200 import Word2Vec
    from bidmach_b200.corpus import zipf_corpus
    from bidmach_b200.word2vec import Opts
    V, D, N = 20_000, 100, 50_000
    toks = dev(zipf_corpus(V, N, 1.0, seed=3, doc_len=500))
    o = Opts(dim=D, vocabSize=V, nSlices=4, iSlice=1, nHeadTerms=1000, doHead=0, lrate=0.01, wsample=1.0, seed=5)
    m = Word2Vec(o).init(N)
    rows = oracle.slice_rows(V, 4, 1000)
    assert m.modelmats[0].shape == (rows, D) and m.modelmats[1].shape == (rows, D)
    m.modelmats[1].copy_(m.modelmats[0].flip(0))
    before = [x.clone() for x in m.modelmats]
    s0 = m.evalbatch([toks], 0, N)
    # the score is that of the slice kernels on the lists the library built
    words, lb, ub, wa, wb = m.wordMats([toks], batch_id=m._batches)
    A, B = m.modelmats[1].cpu().numpy(), m.modelmats[0].cpu().numpy()
    ep = oracle.word2vecEvalPosSlice(D, N, 5, words.cpu().numpy(), lb.cpu().numpy(), ub.cpu().numpy(), A, B, 1, 4, 1000, 4)
    en = oracle.word2vecEvalNegSlice(D, wa.shape[0], 5, 5, wa.cpu().numpy(), wb.cpu().numpy(), A, B, 1, 4, 1000, 4)
    want = oracle.eval_score(ep, en, 5, wb.numel())
    assert abs(s0 - want) <= TOL * abs(want)
    from bidmach_b200 import CUMACHSlice

    def positive_score():
        r = torch.zeros(1, device="cuda")
        assert CUMACHSlice.word2vecEvalPosSlice(D, N, 5, wkeep, lbkeep, ubkeep, m.modelmats[1], m.modelmats[0], r,
                                                1, 4, 1000) == 0
        return r.item()

    wkeep, lbkeep, ubkeep = words.clone(), lb.clone(), ub.clone()
    p0 = positive_score()
    for k in range(3):
        m.dobatch([toks], 0, (k + 1) * N)
    torch.cuda.synchronize()
    assert torch.equal(m.modelmats[0][:1000], before[0][:1000]) and torch.equal(m.modelmats[1][:1000], before[1][:1000])
    assert not torch.equal(m.modelmats[0][1000:], before[0][1000:])
    assert positive_score() > p0        # the slice's own positive pairs became more likely


def test_slice_binders_give_what_the_c_functions_give(oracle):
    """Java_edu_berkeley_bid_CUMACH_word2vecNegSlice / EvalNegSlice through a mock JNIEnv (jcuda.Pointer
    objects with nativePointer + byteOffset) against the oracle."""
    import ctypes as C
    from bidmach_b200 import _lib
    from test_jni_shim import MockJVM
    lib = _lib.load()
    jvm = MockJVM()
    assert lib.JNI_OnLoad(jvm.vm, None) == 0x00010004
    dim, vocab, ncols, nslices, islice, nhead = 100, 3000, 290, 4, 2, 64
    rows = oracle.slice_rows(vocab, nslices, nhead)
    A, B = random_model(rows, dim, 3, scale=0.5)
    WA, WB = conflict_free_neg(ncols, vocab, 5, 5, 4)
    A_ref, B_ref = A.copy(), B.copy()
    oracle.word2vecNegSlice(dim, ncols, 5, 5, WA, WB, A_ref, B_ref, 0.02, 0.5, islice, nslices, nhead, 1)
    dA, dB, dWA, dWB = dev(A), dev(B), dev(WA), dev(WB)
    pA, pB, pWA, pWB = (jvm.pointer(x.data_ptr() - 32, 32) for x in (dA, dB, dWA, dWB))
    assert lib.Java_edu_berkeley_bid_CUMACH_word2vecNegSlice(jvm.env, None, dim, ncols, 5, 5, pWA, pWB, pA, pB,
                                                             0.02, 0.5, islice, nslices, nhead, 1) == 0
    assert rel_err(dA.cpu().numpy() - A, A_ref - A) <= TOL and rel_err(dB.cpu().numpy() - B, B_ref - B) <= TOL
    ret = torch.zeros(1, device="cuda")
    pR = jvm.pointer(ret.data_ptr(), 0)
    assert lib.Java_edu_berkeley_bid_CUMACH_word2vecEvalNegSlice(jvm.env, None, dim, ncols, 5, 5, pWA, pWB, pA, pB,
                                                                 pR, islice, nslices, nhead) == 0
    want = oracle.word2vecEvalNegSlice(dim, ncols, 5, 5, WA, WB, dA.cpu().numpy(), dB.cpu().numpy(), islice,
                                       nslices, nhead)
    assert abs(ret.item() - want) <= TOL * abs(want)


def test_word2vec_slice_methods_forward_to_the_slice_kernels(oracle):
    """Word2Vec.procPositivesSlice / procNegativesSlice / evalPositivesSlice / evalNegativesSlice
    (Word2Vec.scala:404-467, 491-535): A is modelmats(1) and B modelmats(0), slice count, head size
    and doHead come from the options."""
    from bidmach_b200 import Word2Vec
    from bidmach_b200.word2vec import Opts
    vocab, dim, skip, nslices, islice, nhead = 4000, 100, 5, 4, 2, 30
    o = Opts(dim=dim, vocabSize=vocab, nskip=skip, nSlices=nslices, iSlice=islice, nHeadTerms=nhead, doHead=1)
    m = Word2Vec(o, device=torch.device("cuda", 0))
    rows = oracle.slice_rows(vocab, nslices, nhead)
    assert m.sliceRows() == rows
    A, B = random_model(rows, dim, 11, scale=0.5)
    W, LB, UB = conflict_free_pos(3000, vocab, skip, 5)
    WA, WB = conflict_free_neg(500, vocab, 5, 5, 6)
    A_ref, B_ref = A.copy(), B.copy()
    oracle.word2vecPosSlice(dim, len(W), skip, W, LB, UB, A_ref, B_ref, 0.05, 0.5, islice, nslices, nhead, 1)
    oracle.word2vecNegSlice(dim, len(WA), 5, 5, WA, WB, A_ref, B_ref, 0.02, 0.5, islice, nslices, nhead, 1)
    mats = [dev(B), dev(A)]                       # modelmats(0) = B, modelmats(1) = A
    m.procPositivesSlice(skip, dev(W), dev(LB), dev(UB), mats, 0.05, 0.5, islice)
    m.procNegativesSlice(5, 5, dev(WA), dev(WB), mats, 0.02, 0.5, islice)
    gB, gA = mats[0].cpu().numpy(), mats[1].cpu().numpy()
    assert rel_err(gA - A, A_ref - A) <= TOL and rel_err(gB - B, B_ref - B) <= TOL
    Wr, LBr, UBr = random_pos(2000, vocab, skip, 9)
    WAr, WBr = random_neg(400, vocab, 5, 5, 10)
    want_pos = oracle.word2vecEvalPosSlice(dim, len(Wr), skip, Wr, LBr, UBr, gA, gB, islice, nslices, nhead)
    want_neg = oracle.word2vecEvalNegSlice(dim, len(WAr), 5, 5, WAr, WBr, gA, gB, islice, nslices, nhead)
    got_pos = m.evalPositivesSlice(skip, dev(Wr), dev(LBr), dev(UBr), mats, islice)
    got_neg = m.evalNegativesSlice(5, 5, dev(WAr), dev(WBr), mats, islice)
    assert abs(got_pos - want_pos) <= 1e-5 * abs(want_pos) and abs(got_neg - want_neg) <= 1e-5 * abs(want_neg)
