"""Bit-exact parity of the on-device minibatch preprocessing (subsampling mask,
window bounds, ordered context list, permutation, negative ids) with the CPU
restatement of Word2Vec.wordMats / getnegs, through the C-ABI."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _tokens(n, vocab, seed, oov=20, doc_len=(3, 60)):
    rng = np.random.default_rng(seed)
    t = np.empty((n, 2), np.int32)
    t[:, 0] = np.minimum(rng.zipf(1.3, size=n) - 1, vocab + oov - 1)
    ends = np.cumsum(rng.integers(doc_len[0], doc_len[1], size=n))
    t[:, 1] = np.searchsorted(ends, np.arange(n), side="right")
    return t


def _opts(**kw):
    from bidmach_b200.word2vec import Opts
    o = Opts(dim=100, vocabSize=5000, wsample=1e-3)
    for k, v in kw.items():
        setattr(o, k, v)
    return o


@pytest.mark.parametrize("n,nskip,nneg,nreuse,seed", [(4096, 5, 5, 5, 1), (1000, 3, 10, 5, 2),
                                                      (777, 2, 5, 10, 3), (5000, 5, 5, 1, 4),
                                                      (37, 5, 5, 5, 5)])
def test_wordmats_bit_exact_with_supplied_uniforms(oracle, n, nskip, nneg, nreuse, seed):
    from bidmach_b200 import Word2Vec
    o = _opts(nskip=nskip, nneg=nneg, nreuse=nreuse)
    toks = _tokens(n, o.vocabSize, seed)
    rng = np.random.default_rng(seed + 50)
    us, uw = rng.random(n, dtype=np.float32), rng.random(n, dtype=np.float32)
    up = rng.random((n, 2 * nskip), dtype=np.float32)
    un = rng.random(2 * nskip * n * nneg // nreuse + nneg, dtype=np.float32)
    model = Word2Vec(o).init(n)
    words, lb, ub, wa, wb = model.wordMats(
        [dev(toks)], uniforms={"sample": dev(us), "window": dev(uw), "permute": dev(up), "negs": dev(un)})
    torch.cuda.synchronize()
    o_words, o_lb, o_ub, o_ctx, o_wb, o_wa = oracle.wordmats_gpu_branch(
        toks, dict(vocabSize=o.vocabSize, nskip=nskip, nneg=nneg, nreuse=nreuse, wsample=o.wsample,
                   wexpt=o.wexpt), us, uw, up, un)
    assert np.array_equal(words.cpu().numpy(), o_words)
    assert np.array_equal(lb.cpu().numpy(), o_lb) and np.array_equal(ub.cpu().numpy(), o_ub)
    assert np.array_equal(model.last_contexts.cpu().numpy(), o_ctx)
    assert np.array_equal(wb.cpu().numpy(), o_wb)
    assert np.array_equal(wa.cpu().numpy(), o_wa)
    assert (o_words >= 0).any() and (o_words < 0).any() and len(o_ctx) > 0


@pytest.mark.parametrize("sort_permute", [False, True])
def test_wordmats_builtin_generator_matches_its_cpu_restatement(oracle, sort_permute):
    """No draws supplied: the library generates them (Philox), and shuffles the
    pair list either with its keyed bijection (default, nothing is sorted and
    nothing waits for the host) or by sorting random keys as the reference."""
    from bidmach_b200 import Word2Vec
    n = 3000
    o = _opts(seed=0x1234_5678_9ABC_DEF0, sortPermute=sort_permute)
    toks = _tokens(n, o.vocabSize, 9)
    model = Word2Vec(o).init(n)
    batch_id = 7
    words, lb, ub, wa, wb = model.wordMats([dev(toks)], batch_id=batch_id)
    torch.cuda.synchronize()
    us, uw, up, un = oracle.library_uniforms(o.seed, batch_id, n, o.nskip, 2 * o.nskip * n)
    perm = None
    if not sort_permute:
        up, perm = None, (lambda npairs: oracle.library_permutation(o.seed, batch_id, npairs))
    o_words, o_lb, o_ub, o_ctx, o_wb, o_wa = oracle.wordmats_gpu_branch(
        toks, dict(vocabSize=o.vocabSize, nskip=o.nskip, nneg=o.nneg, nreuse=o.nreuse,
                   wsample=o.wsample, wexpt=o.wexpt), us, uw, up, un, perm)
    assert np.array_equal(words.cpu().numpy(), o_words)
    assert np.array_equal(lb.cpu().numpy(), o_lb) and np.array_equal(ub.cpu().numpy(), o_ub)
    assert np.array_equal(model.last_contexts.cpu().numpy(), o_ctx)
    assert np.array_equal(wb.cpu().numpy(), o_wb) and np.array_equal(wa.cpu().numpy(), o_wa)
    assert wb.numel() == (len(o_ctx) // o.nreuse) * o.nreuse


def test_iflip_and_oov_and_single_sentence(oracle):
    from bidmach_b200 import Word2Vec
    n = 512
    o = _opts(iflip=True, wsample=1.0)  # wsample 1 keeps every in-vocabulary word
    toks = _tokens(n, o.vocabSize, 11)
    toks[:, 1] = 0
    flipped = np.ascontiguousarray(toks[:, ::-1])
    rng = np.random.default_rng(1)
    us, uw = rng.random(n, dtype=np.float32), rng.random(n, dtype=np.float32)
    up = rng.random((n, 10), dtype=np.float32)
    un = rng.random(10 * n + 5, dtype=np.float32)
    model = Word2Vec(o).init(n)
    words, lb, ub, wa, wb = model.wordMats(
        [dev(flipped)], uniforms={"sample": dev(us), "window": dev(uw), "permute": dev(up), "negs": dev(un)})
    o_words, o_lb, o_ub, _, o_wb, o_wa = oracle.wordmats_gpu_branch(
        flipped, dict(vocabSize=o.vocabSize, nskip=5, nneg=5, nreuse=5, wsample=1.0, wexpt=0.75,
                      iflip=True), us, uw, up, un)
    assert np.array_equal(words.cpu().numpy(), o_words)
    assert np.array_equal(lb.cpu().numpy(), o_lb) and np.array_equal(ub.cpu().numpy(), o_ub)
    assert np.array_equal(wb.cpu().numpy(), o_wb) and np.array_equal(wa.cpu().numpy(), o_wa)
    kept = toks[:, 0] < o.vocabSize
    assert np.array_equal(o_words >= 0, kept)


def test_init_model_matches_restatement(oracle):
    from bidmach_b200 import Word2Vec
    o = _opts(dim=100, vocabSize=777, seed=42)
    m = Word2Vec(o).init(64)
    want = oracle.library_init_model(42, 100, 777)
    assert np.array_equal(m.modelmats[0].cpu().numpy(), want)
    assert float(m.modelmats[1].abs().max()) == 0.0
    assert abs(float(m.modelmats[0].mean())) < 1e-4 and float(m.modelmats[0].abs().max()) <= 0.5 / 100


@pytest.mark.parametrize("n,nskip,nneg,nreuse,wsample,seed", [(4096, 5, 5, 5, 1e-3, 1), (1000, 3, 10, 5, 1.0, 2),
                                                              (777, 2, 5, 10, 1e-3, 3), (5000, 5, 5, 1, 1.0, 4),
                                                              (37, 5, 5, 5, 1.0, 5), (200_000, 5, 5, 5, 1.0, 6)])
def test_minibatch_calls_build_the_same_lists_without_the_ordered_pair_list(n, nskip, nneg, nreuse, wsample, seed):
    """w2v_dobatch / w2v_evalbatch never write the ordered pair list: the thread of a centre sends
    each of its contexts to the place the inverse of the keyed bijection gives its pair.  WB and WA
    must equal, bit for bit, what w2v_wordmats (ordered list, then shuffle, then negatives) builds
    for the same minibatch and batch id."""
    import ctypes as C
    from bidmach_b200 import _lib, Word2Vec
    o = _opts(nskip=nskip, nneg=nneg, nreuse=nreuse, wsample=wsample, lrate=0.0, seed=seed)
    toks = dev(_tokens(n, o.vocabSize, seed))
    m = Word2Vec(o).init(n)
    lib = _lib.load()
    for call in ("train", "score"):
        if call == "train":
            m.dobatch([toks], 0, n)
        else:
            m.evalbatch([toks], 0, n)
        b = _lib.W2VBuffers()
        assert lib.w2v_buffers(m._ctx, C.byref(b)) == 0
        assert not b.contexts                     # no ordered list was written
        g = b.ngroups
        from bidmach_b200.word2vec import _view_i32
        wb_fused = _view_i32(b.WB, g * nreuse, m.device).clone()
        wa_fused = _view_i32(b.WA, g * nneg, m.device).clone()
        words, lb, ub, wa, wb = m.wordMats([toks], batch_id=m._batches)
        assert wa.shape[0] == g
        assert torch.equal(wb.reshape(-1), wb_fused) and torch.equal(wa.reshape(-1), wa_fused)
        assert m.last_contexts.numel() == b.npairs
