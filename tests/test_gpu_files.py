"""Training from corpus files and checkpoints on disk (GPU)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _opts(**kw):
    from bidmach_b200.word2vec import Opts
    o = Opts(dim=100, vocabSize=2000, wsample=1e-3, lrate=0.05, seed=3)
    for k, v in kw.items():
        setattr(o, k, v)
    return o


def test_training_from_files_equals_training_from_memory(tmp_path):
    """The same tokens through FileSource (three .imat.lz4 files of uneven length,
    minibatches stitched across the file boundaries) and through MatSource."""
    from bidmach_b200 import Learner, MatSource, Word2Vec, matio
    from bidmach_b200.corpus import zipf_corpus
    from bidmach_b200.filesource import FileSource, FileSourceOpts, simpleEnum
    from bidmach_b200.learner import LearnerOpts
    toks = zipf_corpus(2000, 26_000, 1.0, seed=5, doc_len=40)
    pat = str(tmp_path / "train%05d.imat.lz4")
    for i, (lo, hi) in enumerate([(0, 9_500), (9_500, 11_000), (11_000, 26_000)]):
        matio.saveTokens(pat % i, toks[lo:hi])
    lo = LearnerOpts(npasses=1)
    a = Learner(FileSource(FileSourceOpts(fnames=simpleEnum(pat), batchSize=2000)), Word2Vec(_opts()), lo).train()
    b = Learner(MatSource(toks, 2000), Word2Vec(_opts()), lo).train()
    a.datasource.close()
    assert a.samplist == b.samplist and len(a.reslist) == len(b.reslist) >= 2
    # same minibatches, same draws; only the order of the atomic additions differs (two
    # runs from memory agree with each other to a cosine of 0.993 at this learning rate)
    assert np.allclose(a.reslist, b.reslist, rtol=2e-3)
    for x, y in zip(a.model.modelmats, b.model.modelmats):
        cos = torch.nn.functional.cosine_similarity(x.flatten(), y.flatten(), dim=0)
        assert float(cos) > 0.98
    fs = FileSource(FileSourceOpts(fnames=simpleEnum(pat), batchSize=2000))
    k = 0
    while fs.hasNext():
        assert np.array_equal(fs.next()[0], toks[2000 * k: 2000 * (k + 1)])
        k += 1
    fs.close()
    assert k == 13


def test_checkpoint_round_trip_keeps_the_score(tmp_path):
    from bidmach_b200 import Word2Vec
    from bidmach_b200.corpus import zipf_corpus
    n = 4000
    toks = zipf_corpus(2000, 2 * n, 1.0, seed=6, doc_len=40)
    m = Word2Vec(_opts()).init(n)
    m.dobatchg([toks[:n]], 0, n)
    m.dobatchg([toks[n:]], 0, 2 * n)
    d = str(tmp_path / "model") + "/"
    m.save(d)
    m2 = Word2Vec(_opts(dim=7, vocabSize=11)).load(d)        # the checkpoint's options win
    assert (m2.opts.dim, m2.opts.vocabSize, m2.opts.seed) == (100, 2000, 3)
    assert all(torch.equal(x, y) for x, y in zip(m.modelmats, m2.modelmats))
    dt = torch.from_numpy(toks[:n]).cuda()
    s1 = m.evalbatch([dt], 0, n)
    m3 = Word2Vec(_opts()).init(n)
    m3.load(d)
    m3._batches = m._batches - 1                             # same draw counter as the call above
    assert m3.evalbatch([dt], 0, n) == pytest.approx(s1, rel=1e-6)


def test_learner_checkpoints_and_resumes(tmp_path):
    """checkPointFile / checkPointInterval / keepCheckPoints and loadCheckPoint
    (Learner.scala:242-249, 258-259, 397-425) with real checkpoint directories."""
    import os

    from bidmach_b200 import Learner, MatSource, Word2Vec
    from bidmach_b200.corpus import zipf_corpus
    from bidmach_b200.learner import LearnerOpts
    toks = zipf_corpus(2000, 16_000, 1.0, seed=9, doc_len=40)
    pat = str(tmp_path / "w2v%03d") + "/"
    lo = LearnerOpts(npasses=1, checkPointFile=pat, checkPointInterval=0.3, keepCheckPoints=1)
    a = Learner(MatSource(toks, 2000), Word2Vec(_opts()), lo).train()
    kept = sorted(p.name for p in tmp_path.iterdir())
    assert kept == ["w2v002", "w2v003"]                       # 0 and 1 were dropped, 3 is the final one
    assert sorted(os.listdir(tmp_path / "w2v003")) == ["modelmat00.lz4", "modelmat01.lz4", "options.json"]
    b = Learner(MatSource(toks, 2000), Word2Vec(_opts()), LearnerOpts(npasses=1, checkPointFile=pat))
    b.init()
    assert b.loadCheckPoint() and b.opts.nextCheckPoint == 4
    assert all(torch.equal(x, y) for x, y in zip(a.model.modelmats, b.model.modelmats))
