"""Host logic: minibatch schedule, data source dealing, corpora, Philox, and the
multi-rank averaging over a gloo group (CPU, world size 2)."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    """A TCP port nobody listens on right now, for a gloo rendezvous on 127.0.0.1."""
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def test_eval_schedule_matches_learner_nextpass(oracle):
    from bidmach_b200.learner import _scala_mod
    # (istep - 1) % evalStep == 0 with Scala's truncated remainder: 1, 12, 23, ...
    steps = [i for i in range(40) if _scala_mod(i - 1, 11) == 0]
    assert steps == [1, 12, 23, 34]
    assert not oracle.is_eval_step(0, 11, True) and oracle.is_eval_step(1, 11, True)
    assert oracle.is_eval_step(5, 11, False) and not oracle.is_eval_step(0, 11, False)


def test_learning_rate_schedule(oracle):
    assert oracle.lrate_at(1e-3, 0.5, 100000, 100000) == np.float32(1e-3)
    assert abs(float(oracle.lrate_at(1e-3, 0.5, 400000, 100000)) - 0.5e-3) < 1e-9
    assert oracle.eval_score(-10.0, -20.0, 5, 7) == pytest.approx((-10.0 - 4.0) / 7)


def test_matsource_deals_minibatches_round_robin():
    from bidmach_b200.learner import MatSource
    toks = np.arange(2 * 1050, dtype=np.int32).reshape(1050, 2)
    s = MatSource(toks, 100)
    sizes = []
    while s.hasNext():
        sizes.append(s.next()[0].shape[0])
    assert sizes == [100] * 10 + [50]
    a, b = MatSource(toks, 100, 0, 2), MatSource(toks, 100, 1, 2)
    ga, gb = [], []
    while a.hasNext():
        ga.append(int(a.next()[0][0, 0]) // 200)
    while b.hasNext():
        gb.append(int(b.next()[0][0, 0]) // 200)
    assert ga == [0, 2, 4, 6, 8] and gb == [1, 3, 5, 7, 9]   # ragged 11th batch dropped for both
    assert a.nbatches == b.nbatches == 5


class _FakeModel:
    def __init__(self):
        self.calls, self.ncols = [], 100

    def init(self, ncols):
        self.ncols = ncols

    def dobatchg(self, mats, ipass, pos):
        self.calls.append(("train", pos, mats[0].shape[0]))
        return 0

    def evalbatchg(self, mats, ipass, pos):
        self.calls.append(("eval", pos, mats[0].shape[0]))
        return -1.0


def test_learner_replays_the_reference_schedule():
    from bidmach_b200.learner import Learner, LearnerOpts, MatSource
    toks = np.zeros((1450, 2), np.int32)
    m = _FakeModel()
    Learner(MatSource(toks, 100), m, LearnerOpts(npasses=2, evalStep=11)).train()
    kinds = [c[0] for c in m.calls]
    # istep 0 trains, 1 scores, 2 trains and is scored afterwards (the training score,
    # (istep - 1) % evalStep == 1), 3..11 train, 12 scores, 13 trains + training score, 14 (last) scores
    one_pass = ["train", "eval", "train", "eval"] + ["train"] * 9 + ["eval", "train", "eval", "eval"]
    assert kinds == one_pass * 2
    assert [c[1] for c in m.calls][:4] == [100, 200, 300, 300]      # `here` advances by batchSize
    assert m.calls[16][2] == 50                                      # the short last batch still arrives
    assert [c[1] for c in m.calls][17] == 1600                       # and `here` keeps counting in pass 2


def test_corpora_are_seeded_and_ranked():
    from bidmach_b200.corpus import TopicCorpus, zipf_corpus
    a = zipf_corpus(5000, 20000, 1.0, seed=3, doc_len=100)
    b = zipf_corpus(5000, 20000, 1.0, seed=3, doc_len=100)
    assert a.dtype == np.int32 and a.shape == (20000, 2) and np.array_equal(a, b)
    assert not np.array_equal(a, zipf_corpus(5000, 20000, 1.0, seed=4, doc_len=100))
    counts = np.bincount(a[:, 0], minlength=5000)
    assert counts[0] > counts[10] > counts[200] and a[:, 0].max() < 5000
    assert np.array_equal(a[:, 1], np.arange(20000) // 100)
    tc = TopicCorpus(2000, 20, seed=1, doc_len=50, rank_sample_docs=400)
    x, y = tc.tokens(5, 40), tc.tokens(5, 40)
    assert np.array_equal(x, y) and x.shape == (2000, 2) and x[:, 0].max() < 2000
    assert np.array_equal(np.unique(x[:, 1]), np.arange(5, 45))
    c = np.bincount(tc.tokens(100, 400)[:, 0], minlength=2000)
    assert c[:100].sum() > c[1000:1100].sum()                        # low ids are the frequent ones
    # topical structure: a document concentrates on few words compared with the corpus
    doc = tc.tokens(0, 1)[:, 0]
    assert len(np.unique(doc)) < 50


def test_philox_known_answers(oracle):
    """Known-answer vectors of Philox4x32-10 from the generator's publication."""
    z = np.zeros(1, np.uint32)
    out = oracle.philox4x32_10(z, z, z, z, 0, 0)
    assert [int(x[0]) for x in out] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    f = np.full(1, 0xFFFFFFFF, np.uint32)
    out = oracle.philox4x32_10(f, f, f, f, 0xFFFFFFFF, 0xFFFFFFFF)
    assert [int(x[0]) for x in out] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    out = oracle.philox4x32_10(np.array([0x243F6A88], np.uint32), np.array([0x85A308D3], np.uint32),
                               np.array([0x13198A2E], np.uint32), np.array([0x03707344], np.uint32),
                               0xA4093822, 0x299F31D0)
    assert [int(x[0]) for x in out] == [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]
    u = oracle.u01(np.array([0, 0xFFFFFFFF, 0x80000000], np.uint32))
    assert u[0] == 0.0 and u[1] < 1.0 and u[2] == 0.5


def _avg_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bidmach_b200.word2vec import Word2Vec
    m = Word2Vec.__new__(Word2Vec)          # no device needed for the exchange itself
    m.modelmats = [torch.full((6, 4), float(rank + 1)), torch.arange(24.0).view(6, 4) * (rank + 1)]
    m.mergeModelFn()
    q.put((rank, m.modelmats[0].clone(), m.modelmats[1].clone()))
    dist.barrier()
    dist.destroy_process_group()


def _slice_head_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bidmach_b200.word2vec import Opts, Word2Vec
    m = Word2Vec.__new__(Word2Vec)
    m.opts = Opts(nSlices=world, iSlice=rank, nHeadTerms=2)
    m.modelmats = [torch.full((6, 4), float(rank + 1)), torch.arange(24.0).view(6, 4) * (rank + 1)]
    m.mergeHeadFn()
    q.put((rank, m.modelmats[0].clone(), m.modelmats[1].clone()))
    dist.barrier()
    dist.destroy_process_group()


def test_merge_head_averages_only_the_head_rows_of_vocabulary_slices():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_slice_head_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict((r, (a, b)) for r, a, b in (q.get(timeout=120) for _ in range(world)))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank in range(world):
        m0, m1 = got[rank]
        assert torch.allclose(m0[:2], torch.full((2, 4), 1.5)) and torch.allclose(m0[2:], torch.full((4, 4), rank + 1.0))
        base = torch.arange(24.0).view(6, 4)
        assert torch.allclose(m1[:2], base[:2] * 1.5) and torch.allclose(m1[2:], base[2:] * (rank + 1))


def test_merge_model_averages_both_matrices_over_a_gloo_group():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_avg_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, m0, m1 in got:
        assert torch.allclose(m0, torch.full((6, 4), 1.5))
        assert torch.allclose(m1, torch.arange(24.0).view(6, 4) * 1.5)


def _par_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bidmach_b200.learner import LearnerOpts, MatSource, ParLearner

    class M(_FakeModel):
        def __init__(self):
            super().__init__()
            self.modelmats = [torch.full((3, 2), float(rank)), torch.zeros(3, 2)]
            self.merges = 0

        def dobatchg(self, mats, ipass, pos):
            self.modelmats[0] += 1.0 + rank
            return super().dobatchg(mats, ipass, pos)

        def mergeModelFn(self, group=None):
            self.merges += 1
            for t in self.modelmats:
                dist.all_reduce(t)
                t /= world

    toks = np.zeros((2100, 2), np.int32)
    m = M()
    ParLearner(MatSource(toks, 100, rank, world), m, LearnerOpts(npasses=1, evalStep=11, syncStep=2)).train()
    q.put((rank, m.merges, len(m.calls), m.modelmats[0].clone()))
    dist.barrier()
    dist.destroy_process_group()


def test_parlearner_syncs_every_syncstep_and_replicas_agree():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_par_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted((q.get(timeout=120) for _ in range(world)), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # 21 batches -> 20 usable, 10 per rank; istep 1 and the last are eval-only: 8 train steps, 4 syncs;
    # istep 2 is also scored after training (the training score): 11 model calls
    assert got[0][1] == got[1][1] == 4 and got[0][2] == got[1][2] == 11
    assert torch.equal(got[0][3], got[1][3])


def test_parlearner_overlapped_exchange_order():
    """overlapSync: the exchange starts after every syncStep-th training minibatch
    and is folded in right after the next one (or at the end of training)."""
    from bidmach_b200.learner import LearnerOpts, MatSource, ParLearner

    class M(_FakeModel):
        def __init__(self):
            super().__init__()
            self.log = []

        def dobatchg(self, mats, ipass, pos):
            self.log.append("train")
            return 0

        def evalbatchg(self, mats, ipass, pos):
            self.log.append("eval")
            return 0.0

        def startMerge(self, group=None):
            self.log.append("start")

        def finishMerge(self, defer=False):
            self.log.append("finish")

    m = M()
    toks = np.zeros((700, 2), np.int32)
    ParLearner(MatSource(toks, 100), m, LearnerOpts(npasses=1, evalStep=11, syncStep=2, overlapSync=True)).train()
    # minibatches: train, eval, train (+ its training score), train, train, train, eval(last)
    assert m.log == ["train", "finish", "eval", "train", "start", "eval", "train", "finish", "train", "start",
                     "train", "finish", "eval", "finish"]


def test_merge_head_length_follows_the_reference_formula():
    """Word2Vec.scala:548: headlen = max(opts.headlen, opts.headlen << trailingZeros(istep)),
    everything when istep == 0, never more than the vocabulary; Int arithmetic."""
    from bidmach_b200.word2vec import Word2Vec
    f = Word2Vec.mergeHeadLen
    V = 1_000_000
    assert f(10000, 0, V) == V
    assert [f(10000, k, V) for k in (1, 2, 3, 4, 6, 8, 12, 64)] == [10000, 20000, 10000, 40000, 20000, 80000,
                                                                   40000, 640000]
    assert f(10000, 128, V) == V and f(10000, 1 << 10, V) == V
    assert f(10000, 8, 50_000) == 50_000
    # 10000 << 18 overflows Int to a negative number, so max() falls back to headlen;
    # a shift count of 32 wraps to 0
    assert f(10000, 1 << 18, 1 << 40) == 10000
    assert f(10000, 1 << 32, 1 << 40) == 10000
    assert f(10000, 1 << 17, 1 << 40) == 10000 << 17


def _head_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bidmach_b200.word2vec import Opts, Word2Vec
    m = Word2Vec.__new__(Word2Vec)
    m.opts = Opts(vocabSize=12, dim=4, headlen=2)
    m.modelmats = [torch.full((12, 4), float(rank + 1)), torch.full((12, 4), 10.0 * (rank + 1))]
    m.mergeModelFn(None, istep=2)        # head = 2 << 1 = 4 rows
    q.put((rank, m.modelmats[0].clone(), m.modelmats[1].clone()))
    dist.barrier()
    dist.destroy_process_group()


def test_merge_model_with_istep_averages_only_the_head_rows():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_head_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted((q.get(timeout=120) for _ in range(world)), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, m0, m1 in got:
        assert torch.allclose(m0[:4], torch.full((4, 4), 1.5)) and torch.allclose(m1[:4], torch.full((4, 4), 15.0))
        assert torch.equal(m0[4:], torch.full((8, 4), float(rank + 1)))       # the tail stays local
        assert torch.equal(m1[4:], torch.full((8, 4), 10.0 * (rank + 1)))


def test_parlearner_head_sync_counts_every_round_like_the_reference():
    """headSync: ParLearner's istep grows by the number of replicas per round
    (scoring rounds included) and sync k is handed istep / syncStep
    (Learner.scala:654-655)."""
    from bidmach_b200.learner import LearnerOpts, MatSource, ParLearner

    class M(_FakeModel):
        def __init__(self):
            super().__init__()
            self.isteps = []

        def mergeModelFn(self, group=None, istep=0):
            self.isteps.append(istep)

    m = M()
    toks = np.zeros((900, 2), np.int32)
    ParLearner(MatSource(toks, 100), m, LearnerOpts(npasses=1, syncStep=2, headSync=True)).train()
    # one replica: istep = 1..9, syncs when istep % 2 == 0 with istep / 2
    assert m.isteps == [1, 2, 3, 4]


@pytest.mark.parametrize("n", [1, 2, 3, 17, 1000, 65536, 65537, 1_000_003])
def test_keyed_permutation_is_a_bijection(oracle, n):
    """CPU restatement only (the GPU side is compared with it above): every index once."""
    p = oracle.library_permutation(99, 4, n)
    assert p.shape == (n,) and np.array_equal(np.sort(p), np.arange(n))
    if n >= 1000:
        assert abs(np.corrcoef(np.arange(n), p)[0, 1]) < 0.05     # no trace of the input order
        assert (p == np.arange(n)).mean() < 0.01
        assert not np.array_equal(p, oracle.library_permutation(99, 5, n))   # another minibatch, another shuffle


def test_keyed_permutation_known_answers(oracle):
    """Frozen values: the shuffle is part of the library's reproducible behaviour
    (seed, minibatch number -> permutation), so a change of the algorithm must show."""
    assert oracle.library_permutation(99, 4, 1000)[:12].tolist() == [901, 489, 480, 393, 865, 397, 859, 141,
                                                                   978, 308, 64, 102]
    assert oracle.library_permutation(0x123456789ABCDEF0, 7, 5_985_887)[:8].tolist() == [
        5068001, 3494612, 1389536, 5787168, 2465857, 5956610, 135992, 4957205]


def test_learner_checkpoints_as_the_reference(tmp_path):
    """Learner.scala:242-249, 258-259: a checkpoint whenever ipass + progress passes the next
    multiple of checkPointInterval, the one keepCheckPoints back deleted, a last one at the end."""
    from bidmach_b200.learner import Learner, LearnerOpts, MatSource

    class M(_FakeModel):
        def __init__(self):
            super().__init__()
            self.saved, self.deleted = [], []

        def save(self, f):
            self.saved.append(f)

        def delete(self, f):
            self.deleted.append(f)

    m = M()
    toks = np.zeros((1000, 2), np.int32)
    pat = str(tmp_path / "ck%02d") + "/"
    Learner(MatSource(toks, 100), m, LearnerOpts(npasses=1, checkPointFile=pat, checkPointInterval=0.25,
                                                 keepCheckPoints=2)).train()
    # progress 0.1, 0.2, ... 1.0: checkpoints when it passes 0.25, 0.5, 0.75, then the final one
    assert m.saved == [pat % k for k in range(4)]
    assert m.deleted == [pat % 0]


def test_checkpoint_files_can_be_deleted(tmp_path):
    from bidmach_b200 import modelio
    d = str(tmp_path / "ck") + "/"
    modelio.saveModel(d, {"dim": 4}, [np.zeros((3, 4), np.float32), np.ones((3, 4), np.float32)])
    assert (tmp_path / "ck" / "modelmat01.lz4").exists()
    modelio.deleteModel(d)
    assert not (tmp_path / "ck").exists()


def test_learner_progress_log(tmp_path):
    """One JSON object per progress line: the fields of the reference's log line."""
    import json

    from bidmach_b200.learner import Learner, LearnerOpts, MatSource
    log = tmp_path / "progress.jsonl"
    toks = np.zeros((3000, 2), np.int32)
    Learner(MatSource(toks, 100), _FakeModel(), LearnerOpts(npasses=1, pstep=0.25, logFile=str(log))).train()
    rows = [json.loads(l) for l in open(log)]
    assert [round(r["pct"]) for r in rows] == [25, 50, 75, 100]
    assert all(r["val"] == -1.0 and r["words_per_s"] > 0 and r["pass"] == 0 for r in rows)


def test_map_indx_names_the_rows_the_slices_store(oracle):
    """Word2Vec.mapIndx (Word2Vec.scala:665-672) against the layout the slice kernels use."""
    from bidmach_b200 import Word2Vec
    vocab, nrows = 1000, 7
    ids = np.arange(vocab, dtype=np.float32).reshape(-1, 1)
    for nslices, islice, nhead in ((4, 1, 20), (3, 0, 0), (8, 5, 16), (2, 1, 50)):
        stored = oracle.slice_of_model(ids, islice, nslices, nhead)
        rows = oracle.slice_rows(vocab, nslices, nhead)
        seen = 0
        for w in range(vocab):
            m, off, mine, head = Word2Vec.mapIndx(w, islice, nslices, nhead, rows, nrows)
            assert head == (w < nhead) and mine == (w >= nhead and w % nslices == islice)
            if mine or head:
                assert m == 0 and off % nrows == 0 and stored[off // nrows, 0] == w
                seen += 1
        assert seen == nhead + len([w for w in range(nhead, vocab) if w % nslices == islice])
        # several blocks of maxCols rows each, as the reference lays a large slice out
        m, off, _, _ = Word2Vec.mapIndx(nhead + 5 * nslices + islice, islice, nslices, nhead, 4, nrows)
        assert (m, off) == ((nhead + 5) // 4, nrows * ((nhead + 5) % 4))
