"""Edge cases of the whole-minibatch calls (w2v_dobatch / w2v_evalbatch) through
the host mirror: empty pair sets, one-token minibatches, out-of-vocabulary
text, short windows, minibatches of the wrong length."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _model(n, **kw):
    from bidmach_b200 import Word2Vec
    from bidmach_b200.word2vec import Opts
    o = Opts(dim=100, vocabSize=500, wsample=1.0, lrate=0.01, seed=1)
    for k, v in kw.items():
        setattr(o, k, v)
    return Word2Vec(o).init(n)


def _toks(n, vocab, seed=0, doc=20):
    rng = np.random.default_rng(seed)
    t = np.empty((n, 2), np.int32)
    t[:, 0] = rng.integers(0, vocab, n)
    t[:, 1] = np.arange(n) // doc
    return t


def test_all_out_of_vocabulary_minibatch_is_a_no_op():
    m = _model(256)
    before = [x.clone() for x in m.modelmats]
    toks = _toks(256, 500)
    toks[:, 0] += 1000                      # every id >= vocabSize
    assert m.dobatchg([toks], 0, 256) == 0
    assert m.evalbatchg([toks], 0, 256) == 0.0
    assert all(torch.equal(a, b) for a, b in zip(before, m.modelmats))


def test_one_token_per_sentence_yields_no_pairs():
    m = _model(128)
    toks = _toks(128, 500, doc=1)           # every window is clipped to the token itself
    assert m.dobatchg([toks], 0, 128) == 0
    words, lb, ub, wa, wb = m.wordMats([torch.from_numpy(toks).cuda()])
    assert int(lb.abs().max()) == 0 and int(ub.abs().max()) == 0 and wa.numel() == 0 and wb.numel() == 0


def test_single_token_minibatch_and_fewer_pairs_than_nreuse():
    m = _model(1)
    assert m.dobatchg([_toks(1, 500)], 0, 1) == 0
    m3 = _model(2)                          # two pairs < nreuse: no group, positives still train
    before = m3.modelmats[1].clone()
    toks = _toks(2, 500, seed=3, doc=3)
    n = m3.dobatchg([toks], 0, 2)
    assert n == 2
    words, lb, ub, wa, wb = m3.wordMats([torch.from_numpy(toks).cuda()])
    assert wa.numel() == 0
    assert not torch.equal(before, m3.modelmats[1]) or float(m3.modelmats[0].abs().sum()) > 0


def test_minibatch_of_another_length_is_skipped_like_the_reference():
    m = _model(200)
    before = [x.clone() for x in m.modelmats]
    assert m.dobatchg([_toks(150, 500)], 0, 150) == 0
    m.dobatch([torch.from_numpy(_toks(150, 500)).cuda()], 0, 150)
    assert m.evalbatch([torch.from_numpy(_toks(150, 500)).cuda()], 0, 150) == 0.0
    assert all(torch.equal(a, b) for a, b in zip(before, m.modelmats))


@pytest.mark.parametrize("nskip,nneg,nreuse", [(2, 5, 5), (3, 10, 5), (5, 5, 10), (5, 5, 1)])
def test_pipeline_runs_for_every_supported_shape(oracle, nskip, nneg, nreuse):
    n = 3000
    m = _model(n, nskip=nskip, nneg=nneg, nreuse=nreuse, dim=300)
    toks = _toks(n, 500, seed=nskip, doc=37)
    dt = torch.from_numpy(toks).cuda()
    s0 = m.evalbatch([dt], 0, n)
    # A is zero, so every dot is 0; the positive sum covers the few pairs the grouping drops too
    assert s0 == pytest.approx(2 * np.log(0.5), abs=2e-3)
    pairs = m.dobatchg([toks], 0, n)
    words, lb, ub, wa, wb = m.wordMats([dt])
    assert int(ub.max()) <= nskip and int(lb.min()) >= -nskip
    assert pairs > 0
    assert wa.shape[1] == nneg and wb.shape[1] == nreuse
    assert wb.shape[0] == wa.shape[0] == m.last_contexts.numel() // nreuse   # this call drew its own windows
    for _ in range(7):
        m.dobatch([dt], 0, n)
    assert m.evalbatch([dt], 0, n) > s0 + 0.1                   # training on it raises its score
    assert torch.isfinite(m.modelmats[0]).all() and torch.isfinite(m.modelmats[1]).all()


def test_unsupported_options_are_refused():
    from bidmach_b200 import Word2Vec
    from bidmach_b200.word2vec import Opts
    with pytest.raises(RuntimeError):
        Word2Vec(Opts(dim=100, vocabSize=100, nneg=7, nreuse=3)).init(64)
    with pytest.raises(NotImplementedError):
        Word2Vec(Opts(nSlices=2, dualMode=True))
    with pytest.raises(ValueError):
        Word2Vec(Opts(nSlices=2, iSlice=2))
    with pytest.raises(RuntimeError):
        Word2Vec(Opts(useGPU=False))


def test_row_probe_leaves_the_model_unchanged():
    """The benchmark's row-traffic probe (a library of its own, libw2vrowprobe.so): zeros added
    with the update kernel's reductions, or rows read; the model must come out bit for bit as it
    went in."""
    import ctypes as C
    import os
    from bidmach_b200 import _lib
    n = 3000
    m = _model(n, dim=300)
    toks = torch.from_numpy(_toks(n, 500, seed=4, doc=37)).cuda()
    m.dobatch([toks], 0, n)                      # non-trivial matrices
    _, _, _, wa, wb = m.wordMats([toks], batch_id=9)
    before = [x.clone() for x in m.modelmats]
    probe = C.CDLL(os.path.join(os.path.dirname(_lib.LIB_PATH), "libw2vrowprobe.so"))
    probe.w2v_rowprobe.argtypes = [C.c_int] * 4 + [C.c_void_p] * 4 + [C.c_int, C.c_void_p]
    args = (300, wa.shape[0], 5, 5, wa.data_ptr(), wb.data_ptr(), m.modelmats[1].data_ptr(), m.modelmats[0].data_ptr())
    for mode in (0, 1):
        assert probe.w2v_rowprobe(*args, mode, m._stream()) == 0
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(before, m.modelmats))
    assert probe.w2v_rowprobe(*args, 7, m._stream()) == 1


def test_jni_binders_of_the_whole_minibatch_calls():
    """Java_edu_berkeley_bid_CUMACH_w2v*: create, initialise, train and score one minibatch
    through the symbols a JVM would bind (null jcuda.Pointer objects cannot carry an address,
    so the pointers go through a mock JNIEnv as in tests/test_jni_shim.py)."""
    import ctypes as C

    from bidmach_b200 import _lib
    from test_jni_shim import MockJVM
    lib = _lib.load()
    jvm = MockJVM()
    assert lib.JNI_OnLoad(jvm.vm, None) == 0x00010004
    n, V, D = 2000, 500, 100
    h = lib.Java_edu_berkeley_bid_CUMACH_w2vCreate(jvm.env, None, D, 5, 5, 5, V, 0.75, 1.0, 0.01, 0.5, 0.5,
                                                   0, 0, 0, 7, n)
    assert h != 0
    A = torch.empty(V, D, device="cuda")
    B = torch.empty(V, D, device="cuda")
    toks = torch.from_numpy(_toks(n, V, seed=2, doc=37)).cuda()
    pA, pB, pT = (jvm.pointer(x.data_ptr() - 64, 64) for x in (A, B, toks))   # nativePointer + byteOffset
    assert lib.Java_edu_berkeley_bid_CUMACH_w2vInitModel(jvm.env, None, h, pA, pB) == 0
    torch.cuda.synchronize()
    assert float(A.abs().sum()) == 0.0 and float(B.abs().max()) <= 0.5 / D
    s0 = lib.Java_edu_berkeley_bid_CUMACH_w2vEvalbatch(jvm.env, None, h, pT, pA, pB, 1)
    assert s0 == pytest.approx(2 * np.log(0.5), abs=2e-3)
    for k in range(8):
        assert lib.Java_edu_berkeley_bid_CUMACH_w2vDobatch(jvm.env, None, h, pT, pA, pB, n, 2 + k) == 0
    s1 = lib.Java_edu_berkeley_bid_CUMACH_w2vEvalbatch(jvm.env, None, h, pT, pA, pB, 20)
    assert s1 > s0 + 0.05 and lib.Java_edu_berkeley_bid_CUMACH_w2vLastError(jvm.env, None, h) == 0
    lib.Java_edu_berkeley_bid_CUMACH_w2vDestroy(jvm.env, None, h)
    # unsupported options are refused with a null handle
    assert lib.Java_edu_berkeley_bid_CUMACH_w2vCreate(jvm.env, None, D, 5, 7, 3, V, 0.75, 1.0, 0.01, 0.5, 0.5,
                                                      0, 0, 0, 7, n) == 0


def test_reserved_sms_and_the_pos_event_leave_the_result_alone():
    """w2v_reserve_sms only narrows the negative update's grid and w2v_wait_pos only orders another
    stream after the positive update: a minibatch trained with 48 SMs held back, and a side stream
    waiting on the positive update, gives the score a plain run gives (same seeds, same draws; the
    update order differs, hence a tolerance), and both calls refuse a null context."""
    from bidmach_b200 import _lib
    lib = _lib.load()
    n = 50_000
    toks = torch.from_numpy(_toks(n, 5000, seed=2, doc=40)).cuda()
    scores = []
    for reserve in (0, 48):
        m = _model(n, dim=300, vocabSize=5000, lrate=1e-3, wsample=1e-3)
        m.reserveSMs(reserve)
        side = torch.cuda.Stream()
        for k in range(3):
            m.dobatch([toks], 0, (k + 1) * n)
            assert lib.w2v_wait_pos(m._ctx, side.cuda_stream) == 0
        side.synchronize()
        m.reserveSMs(0)
        scores.append(m.evalbatch([toks], 0, n))
    assert abs(scores[0] - scores[1]) <= 0.01 * abs(scores[0]), scores
    assert np.isfinite(scores[0]) and scores[0] > -1.5
    assert lib.w2v_reserve_sms(None, 4) == 1 and lib.w2v_wait_pos(None, None) == 1
    assert lib.w2v_reserve_sms(m._ctx, -1) == 1
