"""The model exchange of the C-ABI: w2v_comm_* / w2v_allreduce_avg (NCCL, for hosts with one
thread or one process per GPU) and w2v_nvls_average (multimem kernel over symmetric memory).
Argument checking runs anywhere; the single-communicator case needs one GPU; the two-replica
cases need two and are skipped elsewhere."""
import ctypes as C
import os
import socket
import threading

import numpy as np
import pytest
import torch


def _lib():
    from bidmach_b200 import _lib
    return _lib.load()


def test_exchange_entry_points_refuse_bad_arguments_without_touching_a_gpu():
    lib = _lib()
    assert lib.w2v_allreduce_avg(None, None, None, 10, None) == 1
    assert lib.w2v_comm_init_all(0, None, None) == 1
    assert lib.w2v_comm_init_rank(2, 2, None, None) == 1
    assert lib.w2v_comm_register(None, None, 0) == 1
    assert lib.w2v_comm_unique_id(None) == 1
    assert lib.w2v_nvls_average(None, 16, 0, 2, 0, None) == 1          # no buffer
    assert lib.w2v_nvls_average(64, 6, 0, 2, 0, None) == 1             # not whole 16-byte vectors
    assert lib.w2v_nvls_average(68, 16, 0, 2, 0, None) == 1            # misaligned
    assert lib.w2v_nvls_average(64, 16, 2, 2, 0, None) == 1            # rank out of range
    lib.w2v_comm_destroy(None)


@pytest.mark.gpu
def test_single_replica_average_is_the_identity():
    lib = _lib()
    comm = C.c_void_p()
    assert lib.w2v_comm_init_all(1, None, C.byref(comm)) == 0
    x = torch.arange(2 * 40, dtype=torch.float32, device="cuda")
    want = x.clone()
    s = torch.cuda.current_stream().cuda_stream
    assert lib.w2v_comm_register(comm, x.data_ptr(), x.numel() * 4) == 0
    assert lib.w2v_allreduce_avg(comm, x.data_ptr(), x.data_ptr() + 4 * 40, 40, s) == 0
    torch.cuda.synchronize()
    assert torch.equal(x, want)
    lib.w2v_comm_destroy(comm)


@pytest.mark.gpu
def test_two_threads_two_gpus_average_through_the_c_abi():
    """The reference's arrangement (ParLearner: one process, one thread per GPU): communicators from
    w2v_comm_init_all, every thread averages its replica; adjacent and separate matrices."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    lib = _lib()
    comms = (C.c_void_p * 2)()
    assert lib.w2v_comm_init_all(2, None, comms) == 0
    n = 3000
    flat = [torch.full((2 * n,), float(r + 1), device=f"cuda:{r}") for r in range(2)]
    sepA = [torch.full((n,), 10.0 * (r + 1), device=f"cuda:{r}") for r in range(2)]
    sepB = [torch.full((n,), -4.0 * (r + 1), device=f"cuda:{r}") for r in range(2)]
    errs = [None, None]

    def work(r):
        torch.cuda.set_device(r)
        s = torch.cuda.current_stream().cuda_stream
        e1 = lib.w2v_allreduce_avg(comms[r], flat[r].data_ptr(), flat[r].data_ptr() + 4 * n, n, s)
        e2 = lib.w2v_allreduce_avg(comms[r], sepA[r].data_ptr(), sepB[r].data_ptr(), n, s)
        torch.cuda.synchronize()
        errs[r] = (e1, e2)

    ts = [threading.Thread(target=work, args=(r,)) for r in range(2)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert errs == [(0, 0), (0, 0)]
    for r in range(2):
        assert torch.all(flat[r] == 1.5) and torch.all(sepA[r] == 15.0) and torch.all(sepB[r] == -6.0)
    for r in range(2):
        lib.w2v_comm_destroy(comms[r])


@pytest.mark.gpu
def test_exchange_binders_on_one_gpu():
    """w2vCommInitAll / w2vCommOf / w2vAllreduceAvg / w2vCommDestroyAll through a mock JNIEnv: one
    replica, so the average is the identity, and the call lands on the calling thread's stream."""
    from test_jni_shim import MockJVM
    lib = _lib()
    jvm = MockJVM()
    assert lib.JNI_OnLoad(jvm.vm, None) == 0x00010004
    comms = lib.Java_edu_berkeley_bid_CUMACH_w2vCommInitAll(jvm.env, None, 1)
    assert comms != 0
    comm = lib.Java_edu_berkeley_bid_CUMACH_w2vCommOf(jvm.env, None, comms, 0)
    assert comm != 0 and lib.Java_edu_berkeley_bid_CUMACH_w2vCommOf(jvm.env, None, comms, 1) == 0
    A = torch.arange(50, dtype=torch.float32, device="cuda")
    B = -A.clone()
    pA, pB = jvm.pointer(A.data_ptr(), 0), jvm.pointer(B.data_ptr() - 16, 16)
    assert lib.Java_edu_berkeley_bid_CUMACH_w2vAllreduceAvg(jvm.env, None, comm, pA, pB, 50) == 0
    torch.cuda.synchronize()
    assert torch.equal(A, torch.arange(50, dtype=torch.float32, device="cuda")) and torch.equal(B, -A)
    lib.Java_edu_berkeley_bid_CUMACH_w2vCommDestroyAll(jvm.env, None, comms)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nvls_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from bidmach_b200 import Word2Vec
    from bidmach_b200.word2vec import Opts
    m = Word2Vec(Opts(dim=100, vocabSize=5003, seed=rank), device=torch.device("cuda", rank)).init(1000)
    ok = m.enableSymmetric()
    if not ok:
        q.put((rank, "no symmetric memory: " + getattr(m, "_symm_error", "no multicast address")))
    else:
        g = torch.Generator(device="cuda")
        g.manual_seed(100 + rank)
        for mm in m.modelmats:
            mm.copy_(torch.rand(mm.shape, device="cuda", generator=g))
        mine = m._flat.clone()
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        want = torch.stack(gathered).mean(0)
        m.mergeModelFn()                       # blocking form: fence, kernel on all SMs, fence
        torch.cuda.synchronize()
        err1 = float((m._flat - want).abs().max())
        # overlapped form, on a few SMs, with nothing else running: same result from the same start
        m._flat.copy_(mine)
        torch.cuda.synchronize()
        dist.barrier()
        m.startMerge()
        m.finishMerge()
        torch.cuda.synchronize()
        err2 = float((m._flat - want).abs().max())
        q.put((rank, (err1, err2)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_two_replicas_average_in_place_through_the_multicast_mapping():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_nvls_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, res in got:
        if isinstance(res, str):
            pytest.skip(res)
        assert res[0] <= 1e-6 and res[1] <= 1e-6, (rank, res)


def _train_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from bidmach_b200 import Word2Vec
    from bidmach_b200.corpus import TopicCorpus
    from bidmach_b200.learner import LearnerOpts, MatSource, ParLearner
    from bidmach_b200.word2vec import Opts
    V, D, N = 10_000, 100, 100_000
    tc = TopicCorpus(V, 50, s=1.07, alpha=0.1, doc_len=1000, seed=5, rank_sample_docs=2000)
    train, held = tc.tokens(0, 60 * 100), tc.tokens(9000, 300)
    out = {}
    for name, lo in (("blocking_nccl", LearnerOpts(npasses=1, evalStep=1000, syncStep=4, exchange="nccl")),
                     ("overlapped_nvls", LearnerOpts(npasses=1, evalStep=1000, syncStep=4, exchange="auto",
                                                     overlapSync=True))):
        model = Word2Vec(Opts(dim=D, vocabSize=V, lrate=1e-3, seed=3 + 7919 * rank), device=torch.device("cuda", rank))
        lr = ParLearner(MatSource(train, N, rank, world), model, lo)
        lr.train()
        torch.cuda.synchronize()
        dist.barrier()
        scores = lr.predict(MatSource(held, N))
        out[name] = (float(np.mean(scores)), bool(model._mc))
    q.put((rank, out))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_two_replicas_learn_the_same_with_the_overlapped_in_place_average():
    """Data-parallel training over two replicas, averaged every 4 minibatches: the blocking NCCL
    all-reduce against the in-place multimem average that runs beside the next minibatch.  Same
    data, same seeds; held-out score within 1 % and the gain over the untrained score within 10 %."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_train_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    untrained = 2 * np.log(0.5)
    for rank in range(world):
        (blk, _), (ovl, in_place) = got[rank]["blocking_nccl"], got[rank]["overlapped_nvls"]
        if not in_place:
            pytest.skip("no symmetric memory with a multicast mapping on this machine")
        assert blk - untrained > 0.05
        assert abs(ovl - blk) <= 0.01 * abs(blk), (rank, ovl, blk)
        assert abs((ovl - untrained) - (blk - untrained)) <= 0.10 * (blk - untrained), (rank, ovl, blk)


def _slice_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from bidmach_b200 import Word2Vec
    from bidmach_b200.corpus import TopicCorpus
    from bidmach_b200.learner import LearnerOpts, MatSource, ParLearner
    from bidmach_b200.word2vec import Opts
    V, D, N, H = 10_000, 100, 100_000, 500
    tc = TopicCorpus(V, 50, s=1.07, alpha=0.1, doc_len=1000, seed=5, rank_sample_docs=2000)
    train, held = tc.tokens(0, 30 * 100), tc.tokens(9000, 100)
    model = Word2Vec(Opts(dim=D, vocabSize=V, lrate=1e-3, seed=3, nSlices=world, iSlice=rank, nHeadTerms=H),
                     device=torch.device("cuda", rank))
    lr = ParLearner(MatSource(train, N, 0, 1), model, LearnerOpts(npasses=1, evalStep=1000, syncStep=4))
    lr.init()
    before = model.evalbatchg([held], 0, N)
    lr.train(do_init=False)
    model.mergeHeadFn()
    torch.cuda.synchronize()
    after = model.evalbatchg([held], 0, N)
    heads = [model.modelmats[j][:H].clone() for j in range(2)]
    others = [[torch.empty_like(h) for _ in range(world)] for h in heads]
    for h, o in zip(heads, others):
        dist.all_gather(o, h)
    same = all(torch.equal(o[0], o[r]) for o in others for r in range(world))
    rows = model.modelmats[0].shape[0]
    q.put((rank, before, after, same, rows))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_two_vocabulary_slices_train_side_by_side_and_share_their_head():
    """Two GPUs, each one vocabulary slice of a model (nSlices = 2), both fed every minibatch: after
    training and a last head average the head rows are identical on both, each holds only its
    slice's rows, and each slice's held-out score has improved."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_slice_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=600) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, before, after, same, rows in got:
        assert same
        assert rows == 500 + 1 + (10_000 - 500 - 1) // 2
        assert after > before + 0.01, (rank, before, after)
