"""CPU oracle for the Word2Vec SGNS minibatch path -- TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module.  It is used by ``tests/``,
by ``__graft_entry__.smoke()`` and by the CPU-baseline legs of ``bench.py`` as
the checker (or as the thing timed as "the CPU way"), never as the product.

Two back ends behind one interface:

* ``impl="port"``       this repository's C restatement, ``oracle/w2v_oracle.c``
* ``impl="reference"``  the reference's own ``jni/src/BIDMach_CPUMACH.c``,
  compiled unchanged into ``oracle/_ref/libw2vref.so`` by ``oracle/build.py``
  (update kernels only; its eval functions return an uninitialised accumulator,
  BIDMach_CPUMACH.c:379,423, so scoring always uses the port, which restates
  the Scala code networks/Word2Vec.scala:953-1005,1071-1132)

plus numpy restatements of the pieces that are not C in the reference:
the GPU-branch permutation of ``Word2Vec.wordMats`` (networks/Word2Vec.scala:
243-270), the learning-rate schedule of ``dobatch`` (:167-177), the score of
``evalbatch`` (:209), the minibatch schedule of ``Learner.nextPass``
(Learner.scala:173-252) and the Philox4x32-10 generator the CUDA library uses
when the caller supplies no uniform draws.

Parity status: the reference has no test, golden vector or fixture for this
path; the port is pinned against the compiled reference C (bit-exact, see
tests/test_oracle_pinning.py) and against fixtures generated from it
(tests/golden).  Random-number streams and the sort-based permutation come
from BIDMat, which is not part of the reference checkout: parity unpinned for
those, they are compared as deterministic maps of caller-supplied uniforms.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import numpy as np

from . import build as _build

_I = C.POINTER(C.c_int)
_F = C.POINTER(C.c_float)
_D = C.POINTER(C.c_double)


def _ip(a):
    return a.ctypes.data_as(_I)


def _fp(a):
    return a.ctypes.data_as(_F)


_port = None
_ref = None


def port_lib():
    global _port
    if _port is None:
        _port = C.CDLL(_build.build_oracle())
        _port.orc_word2vecEvalPos.restype = C.c_double
        _port.orc_word2vecEvalNeg.restype = C.c_double
        _port.orc_word2vecEvalPosSlice.restype = C.c_double
        _port.orc_word2vecEvalNegSlice.restype = C.c_double
        _port.orc_count_pairs.restype = C.c_int64
        _port.orc_fill_contexts.restype = C.c_int64
    return _port


def ref_lib():
    """The compiled reference, or None when it was never built on this machine."""
    global _ref
    if _ref is None:
        path = _build.build_ref()
        if path is None:
            return None
        _ref = C.CDLL(path)
        _ref.ref_word2vecEvalPos.restype = C.c_double
        _ref.ref_word2vecEvalNeg.restype = C.c_double
    return _ref


def have_reference() -> bool:
    return ref_lib() is not None


def set_threads(n: int) -> int:
    """Fixes the OpenMP team size of both back ends (they share one OpenMP runtime) and returns
    the number of threads a parallel region then really runs with."""
    got = int(port_lib().orc_set_threads(C.c_int(n)))
    ref = ref_lib()
    if ref is not None and hasattr(ref, "ref_set_threads"):
        got = int(ref.ref_set_threads(C.c_int(n)))
    return got


def _i32(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a


def _check_model(M, nrows):
    assert M.dtype == np.float32 and M.flags.c_contiguous and M.size % nrows == 0


# ---------------------------------------------------------------------------
# the four kernels (A, B are float32 arrays of shape [vocab, dim]: one word per row)
# ---------------------------------------------------------------------------

def word2vecPos(nrows, ncols, skip, W, LB, UB, A, B, lrate, vexp, nthreads=1, impl="port"):
    """In-place positive update; CPUMACH.word2vecPos (BIDMach_CPUMACH.c:10-78)."""
    W, LB, UB = _i32(W), _i32(LB), _i32(UB)
    _check_model(A, nrows)
    _check_model(B, nrows)
    args = (C.c_int(nrows), C.c_int(ncols), C.c_int(skip), _ip(W), _ip(LB), _ip(UB), _fp(A), _fp(B),
            C.c_float(lrate), C.c_float(vexp), C.c_int(nthreads))
    if impl == "reference":
        ref_lib().ref_word2vecPos(*args)
    else:
        port_lib().orc_word2vecPos(*args)


def word2vecNeg(nrows, ncols, nwa, nwb, WA, WB, A, B, lrate, vexp, nthreads=1, impl="port"):
    """In-place negative update; CPUMACH.word2vecNeg (BIDMach_CPUMACH.c:186-264)."""
    WA, WB = _i32(WA), _i32(WB)
    _check_model(A, nrows)
    _check_model(B, nrows)
    args = (C.c_int(nrows), C.c_int(ncols), C.c_int(nwa), C.c_int(nwb), _ip(WA), _ip(WB), _fp(A),
            _fp(B), C.c_float(lrate), C.c_float(vexp), C.c_int(nthreads))
    if impl == "reference":
        ref_lib().ref_word2vecNeg(*args)
    else:
        port_lib().orc_word2vecNeg(*args)


def word2vecEvalPos(nrows, ncols, skip, W, LB, UB, A, B, nthreads=1):
    """Word2Vec.evalPosCPU (networks/Word2Vec.scala:953-1005)."""
    W, LB, UB = _i32(W), _i32(LB), _i32(UB)
    return float(port_lib().orc_word2vecEvalPos(
        C.c_int(nrows), C.c_int(ncols), C.c_int(skip), _ip(W), _ip(LB), _ip(UB), _fp(A), _fp(B),
        C.c_int(nthreads)))


def word2vecEvalNeg(nrows, ncols, nwa, nwb, WA, WB, A, B, nthreads=1):
    """Word2Vec.evalNegCPU (networks/Word2Vec.scala:1071-1132)."""
    WA, WB = _i32(WA), _i32(WB)
    return float(port_lib().orc_word2vecEvalNeg(
        C.c_int(nrows), C.c_int(ncols), C.c_int(nwa), C.c_int(nwb), _ip(WA), _ip(WB), _fp(A), _fp(B),
        C.c_int(nthreads)))


def slice_rows(vocab, nslices, nhead):
    """Rows of a slice's matrices: nHeadTerms + 1 + (nfeats - nHeadTerms - 1) / nSlices
    (Word2Vec.init, networks/Word2Vec.scala:106)."""
    return vocab if nslices <= 1 else nhead + 1 + (vocab - nhead - 1) // nslices


def slice_of_model(M, islice, nslices, nhead):
    """The rows of a whole-vocabulary matrix that slice ``islice`` stores, in its own order
    (mapIndx, networks/Word2Vec.scala:665-672): the head, then the ids congruent to islice."""
    vocab = M.shape[0]
    ids = np.arange(vocab)
    mine = ids[(ids >= nhead) & (ids % nslices == islice)]
    out = np.zeros((slice_rows(vocab, nslices, nhead), M.shape[1]), np.float32)
    out[:nhead] = M[:nhead]
    out[(mine - nhead) // nslices + nhead] = M[mine]
    return out


def word2vecPosSlice(nrows, ncols, skip, W, LB, UB, A, B, lrate, vexp, islice, nslices, nhead, do_head=1,
                     nthreads=1, impl="port"):
    """In-place positive update of one vocabulary slice; CPUMACH.word2vecPosSlice
    (BIDMach_CPUMACH.c:90-184).  A, B: the slice's rows, one matrix per side."""
    W, LB, UB = _i32(W), _i32(LB), _i32(UB)
    _check_model(A, nrows)
    _check_model(B, nrows)
    if impl == "reference":
        mats = (C.c_void_p * 2)(B.ctypes.data, A.ctypes.data)     # matrix 2m: context rows, 2m+1: centre rows
        ref_lib().ref_word2vecPosSlice(
            C.c_int(nrows), C.c_int(ncols), C.c_int(skip), _ip(W), _ip(LB), _ip(UB), mats, C.c_int(2),
            C.c_float(lrate), C.c_float(vexp), C.c_int(nthreads), C.c_int(islice), C.c_int(nslices),
            C.c_int(A.shape[0] + 1), C.c_int(nhead), C.c_int(0), C.c_int(do_head))
    else:
        port_lib().orc_word2vecPosSlice(
            C.c_int(nrows), C.c_int(ncols), C.c_int(skip), _ip(W), _ip(LB), _ip(UB), _fp(A), _fp(B),
            C.c_float(lrate), C.c_float(vexp), C.c_int(nthreads), C.c_int(islice), C.c_int(nslices),
            C.c_int(nhead), C.c_int(do_head))


def word2vecNegSlice(nrows, ncols, nwa, nwb, WA, WB, A, B, lrate, vexp, islice, nslices, nhead, do_head=1,
                     nthreads=1, impl="port"):
    """In-place negative update of one vocabulary slice; CPUMACH.word2vecNegSlice
    (BIDMach_CPUMACH.c:267-366)."""
    WA, WB = _i32(WA), _i32(WB)
    _check_model(A, nrows)
    _check_model(B, nrows)
    if impl == "reference":
        mats = (C.c_void_p * 2)(B.ctypes.data, A.ctypes.data)
        ref_lib().ref_word2vecNegSlice(
            C.c_int(nrows), C.c_int(ncols), C.c_int(nwa), C.c_int(nwb), _ip(WA), _ip(WB), mats, C.c_int(2),
            C.c_float(lrate), C.c_float(vexp), C.c_int(nthreads), C.c_int(islice), C.c_int(nslices),
            C.c_int(A.shape[0] + 1), C.c_int(nhead), C.c_int(0), C.c_int(do_head))
    else:
        port_lib().orc_word2vecNegSlice(
            C.c_int(nrows), C.c_int(ncols), C.c_int(nwa), C.c_int(nwb), _ip(WA), _ip(WB), _fp(A), _fp(B),
            C.c_float(lrate), C.c_float(vexp), C.c_int(nthreads), C.c_int(islice), C.c_int(nslices),
            C.c_int(nhead), C.c_int(do_head))


def word2vecEvalPosSlice(nrows, ncols, skip, W, LB, UB, A, B, islice, nslices, nhead, nthreads=1):
    """Word2Vec.evalPosCPUslice (networks/Word2Vec.scala:1007-1068)."""
    W, LB, UB = _i32(W), _i32(LB), _i32(UB)
    return float(port_lib().orc_word2vecEvalPosSlice(
        C.c_int(nrows), C.c_int(ncols), C.c_int(skip), _ip(W), _ip(LB), _ip(UB), _fp(A), _fp(B),
        C.c_int(nthreads), C.c_int(islice), C.c_int(nslices), C.c_int(nhead)))


def word2vecEvalNegSlice(nrows, ncols, nwa, nwb, WA, WB, A, B, islice, nslices, nhead, nthreads=1):
    """Word2Vec.evalNegCPUslice (networks/Word2Vec.scala:1134-1200)."""
    WA, WB = _i32(WA), _i32(WB)
    return float(port_lib().orc_word2vecEvalNegSlice(
        C.c_int(nrows), C.c_int(ncols), C.c_int(nwa), C.c_int(nwb), _ip(WA), _ip(WB), _fp(A), _fp(B),
        C.c_int(nthreads), C.c_int(islice), C.c_int(nslices), C.c_int(nhead)))


def word2vecNegFilt(nrows, ncols, nwords, nwa, nwb, WA, WB, A, B, lrate, vexp):
    """Masked negative update: ids >= nwords act as zero rows and are not written
    (__word2vecNegFilt, jni/src/DNN127.cu:670-823).  The reference has no CPU
    twin of this kernel; numpy restatement, small inputs only."""
    WA = _i32(WA).reshape(ncols, nwa)
    WB = _i32(WB).reshape(ncols, nwb)
    f32 = np.float32
    for c in range(ncols):
        ar = [A[w].copy() if w < nwords else np.zeros(nrows, f32) for w in WA[c]]
        br = [B[w].copy() if w < nwords else np.zeros(nrows, f32) for w in WB[c]]
        g = np.zeros((nwa, nwb), f32)
        for j in range(nwa):
            for k in range(nwb):
                g[j, k] = f32(-lrate) * _sigmoid32(f32(np.dot(ar[j], br[k])))
        for j, w in enumerate(WA[c]):
            if w < nwords:
                sa = f32(math.pow(1 + int(w), vexp))
                A[w] += sum((sa * g[j, k]) * br[k] for k in range(nwb))
        for k, w in enumerate(WB[c]):
            if w < nwords:
                sb = f32(math.pow(1 + int(w), vexp))
                B[w] += sum((sb * g[j, k]) * ar[j] for j in range(nwa))


def _sigmoid32(x):
    if x > 16.0:
        return np.float32(1.0)
    if x < -16.0:
        return np.float32(0.0)
    e = np.float32(math.exp(float(x)))
    return np.float32(e / (np.float32(1.0) + e))


# ---------------------------------------------------------------------------
# preprocessing (Word2Vec.wordMats / getnegs)
# ---------------------------------------------------------------------------

def salpha_of(wsample, vocab):
    """opts.wsample * math.log(nfeats).toFloat  (networks/Word2Vec.scala:150)."""
    return np.float32(np.float32(wsample) * np.float32(math.log(vocab)))


def expt_of(wexpt):
    """1f / (1f - opts.wexpt)  (networks/Word2Vec.scala:139)."""
    return np.float32(np.float32(1.0) / (np.float32(1.0) - np.float32(wexpt)))


def wordmats_bounds(tokens, vocab, nskip, salpha, u_sample, u_window, iflip=False):
    """Subsampling mask and window bounds (networks/Word2Vec.scala:214-241).
    tokens: int32 [ncols, 2] (word id, sentence id per token).  Returns words, lb, ub."""
    tokens = _i32(tokens)
    n = tokens.shape[0]
    words = np.empty(n, np.int32)
    lb = np.empty(n, np.int32)
    ub = np.empty(n, np.int32)
    u1 = np.ascontiguousarray(u_sample, np.float32)
    u2 = np.ascontiguousarray(u_window, np.float32)
    port_lib().orc_wordmats_bounds(C.c_int(n), _ip(tokens), C.c_int(1 if iflip else 0),
                                   C.c_int(vocab), C.c_int(nskip), C.c_float(salpha), _fp(u1),
                                   _fp(u2), _ip(words), _ip(lb), _ip(ub))
    return words, lb, ub


def count_pairs(words, lb, ub):
    words, lb, ub = _i32(words), _i32(lb), _i32(ub)
    return int(port_lib().orc_count_pairs(C.c_int(len(words)), _ip(words), _ip(lb), _ip(ub)))


def ordered_contexts(words, lb, ub):
    """Good context words, centre ascending then offset ascending
    (fill loop of getnegs, networks/Word2Vec.scala:309-330)."""
    words, lb, ub = _i32(words), _i32(lb), _i32(ub)
    n = count_pairs(words, lb, ub)
    ctx = np.empty(max(n, 1), np.int32)
    got = port_lib().orc_fill_contexts(C.c_int(len(words)), _ip(words), _ip(lb), _ip(ub), _ip(ctx),
                                       C.c_int64(n))
    assert got == n
    return ctx[:n]


def context_rows(words, lb, ub, nskip):
    """Row of the 2*nskip x ncols context table each ordered pair comes from, and
    its centre: row r holds offset r - nskip for r < nskip, r - nskip + 1 otherwise
    (skipcol, networks/Word2Vec.scala:138-141)."""
    rows, centres = [], []
    for i in range(len(words)):
        if words[i] < 0:
            continue
        for j in range(lb[i], ub[i] + 1):
            if j != 0 and words[i + j] >= 0:
                rows.append(j + nskip if j < 0 else j + nskip - 1)
                centres.append(i)
    return np.asarray(rows, np.int64), np.asarray(centres, np.int64)


def negative_ids(u, expt, vocab):
    """min(V-1, int(V * u^expt)), power in double (networks/Word2Vec.scala:356)."""
    u = np.ascontiguousarray(u, np.float32)
    out = np.empty(u.size, np.int32)
    port_lib().orc_negative_ids(C.c_int64(u.size), _fp(u), C.c_float(expt), C.c_int(vocab), _ip(out))
    return out


def getnegs(words, lb, ub, nneg, nreuse, vocab, expt, prand, randneg):
    """CPU branch of wordMats (Word2Vec.getnegs, networks/Word2Vec.scala:280-364):
    ordered fill, serial shuffle with doubles `prand`, negatives from `randneg`.
    Returns (trandwords [ngroups, nneg], contextwords [ngroups, nreuse])."""
    ctx = ordered_contexts(words, lb, ub)
    ngroups = len(ctx) // nreuse
    ctx = np.ascontiguousarray(ctx[: ngroups * nreuse])
    pr = np.ascontiguousarray(prand[: ctx.size], np.float64)
    port_lib().orc_shuffle(C.c_int64(ctx.size), _ip(ctx), pr.ctypes.data_as(_D))
    negs = negative_ids(np.asarray(randneg, np.float32)[: ngroups * nneg], expt, vocab)
    return negs.reshape(ngroups, nneg), ctx.reshape(ngroups, nreuse)


def permute_by_keys(ctx, u_keys):
    """GPU branch of wordMats (networks/Word2Vec.scala:254-259): every good pair
    gets the fp32 key (u + 1) - 1, the pairs are sorted by descending key; equal
    keys keep their original order (the order among ties is not defined by the
    reference; a stable sort is this build's definition)."""
    k = (np.asarray(u_keys, np.float32) + np.float32(1.0)) - np.float32(1.0)
    order = np.argsort(-k.astype(np.float64), kind="stable")
    return np.asarray(ctx)[order]


def wordmats_gpu_branch(tokens, opts, u_sample, u_window, u_permute, u_negs, perm=None):
    """Whole wordMats with the GPU branch's permutation.  u_permute is the
    [ncols, 2*nskip] table of draws; when it is None, ``perm`` (an index array,
    see library_permutation) shuffles the ordered list instead.  Returns words,
    lb, ub, contexts (ordered), WB [ngroups, nreuse], WA [ngroups, nneg].
    ``perm`` may also be a function of the pair count."""
    V, nskip = opts["vocabSize"], opts["nskip"]
    words, lb, ub = wordmats_bounds(tokens, V, nskip, salpha_of(opts["wsample"], V), u_sample,
                                    u_window, opts.get("iflip", False))
    ctx = ordered_contexts(words, lb, ub)
    if u_permute is None:
        if callable(perm):
            perm = perm(len(ctx))
        perm = np.asarray(ctx)[np.asarray(perm, np.int64)]
    else:
        rows, centres = context_rows(words, lb, ub, nskip)
        keys = np.asarray(u_permute, np.float32).reshape(len(words), 2 * nskip)[centres, rows]
        perm = permute_by_keys(ctx, keys)
    ngroups = len(ctx) // opts["nreuse"]
    WB = perm[: ngroups * opts["nreuse"]].reshape(ngroups, opts["nreuse"])
    WA = negative_ids(np.asarray(u_negs, np.float32).ravel()[: ngroups * opts["nneg"]],
                      expt_of(opts["wexpt"]), V).reshape(ngroups, opts["nneg"])
    return words, lb, ub, ctx, WB, WA


# ---------------------------------------------------------------------------
# Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy
# as 1, 2, 3", SC'11), vectorised; stream layout as in the CUDA library.
# ---------------------------------------------------------------------------
STREAM_SAMPLE_WINDOW, STREAM_PERMUTE, STREAM_NEGS, STREAM_INIT = 1, 2, 3, 4


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    W0, W1 = 0x9E3779B9, 0xBB67AE85
    c0, c1, c2, c3 = (np.asarray(np.broadcast_arrays(c0, c1, c2, c3)[i], np.uint32).copy()
                      for i in range(4))
    k0, k1 = int(k0) & 0xFFFFFFFF, int(k1) & 0xFFFFFFFF
    lo32 = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = M0 * c0.astype(np.uint64)
        p1 = M1 * c2.astype(np.uint64)
        n0 = ((p1 >> np.uint64(32)).astype(np.uint32)) ^ c1 ^ np.uint32(k0)
        n1 = (p1 & lo32).astype(np.uint32)
        n2 = ((p0 >> np.uint64(32)).astype(np.uint32)) ^ c3 ^ np.uint32(k1)
        n3 = (p0 & lo32).astype(np.uint32)
        c0, c1, c2, c3 = n0, n1, n2, n3
        k0 = (k0 + W0) & 0xFFFFFFFF
        k1 = (k1 + W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def u01(x):
    return (x >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)


def library_uniforms(seed, batch_id, ncols, nskip, n_negs):
    """The draws the CUDA library generates for one minibatch when given none."""
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    b = np.uint32(batch_id & 0xFFFFFFFF)
    i = np.arange(ncols, dtype=np.uint32)
    r = philox4x32_10(i, 0, STREAM_SAMPLE_WINDOW, b, k0, k1)
    sample, window = u01(r[0]), u01(r[1])
    nblk = (2 * nskip + 3) // 4
    perm = np.empty((ncols, nblk * 4), np.float32)
    for blk in range(nblk):
        r = philox4x32_10(i, blk, STREAM_PERMUTE, b, k0, k1)
        for q in range(4):
            perm[:, blk * 4 + q] = u01(r[q])
    perm = np.ascontiguousarray(perm[:, : 2 * nskip])
    nb = (n_negs + 3) // 4
    blk = np.arange(nb, dtype=np.uint64)
    r = philox4x32_10((blk & np.uint64(0xFFFFFFFF)).astype(np.uint32),
                      (blk >> np.uint64(32)).astype(np.uint32), STREAM_NEGS, b, k0, k1)
    negs = np.stack([u01(x) for x in r], axis=1).ravel()[:n_negs]
    return sample, window, perm, negs


def keyed_permutation(n, a, c):
    """Keyed bijection of [0, n) the CUDA library shuffles pair indices with
    when it sorts nothing: four rounds of x = (x*a[r] + c[r]) mod 2^b,
    x ^= x >> ceil(b/2) (b = bit length of n-1, a[r] odd), applied again while
    the value is >= n (cycle walking).  Returns perm with perm[i] = image of i."""
    n = int(n)
    if n < 2:
        return np.zeros(n, np.int64)
    b = int(n - 1).bit_length()
    mask, sh = np.uint64((1 << b) - 1), np.uint64((b + 1) >> 1)
    x = np.arange(n, dtype=np.uint64)
    out = np.empty(n, np.int64)
    todo = np.arange(n)
    while todo.size:
        v = x[todo]
        for r in range(4):
            v = (v * np.uint64(a[r]) + np.uint64(c[r])) & mask
            v ^= v >> sh
        x[todo] = v
        done = v < np.uint64(n)
        out[todo[done]] = v[done].astype(np.int64)
        todo = todo[~done]
    return out


def library_permutation(seed, batch_id, n):
    """keyed_permutation with the constants the CUDA library derives for one
    minibatch: two Philox blocks of the permutation stream, multipliers made odd."""
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    b = np.uint32(batch_id & 0xFFFFFFFF)
    x = philox4x32_10(np.uint32(0), 0, STREAM_PERMUTE, b, k0, k1)
    y = philox4x32_10(np.uint32(1), 0, STREAM_PERMUTE, b, k0, k1)
    a = [int(np.asarray(v).ravel()[0]) | 1 for v in x]
    c = [int(np.asarray(v).ravel()[0]) for v in y]
    return keyed_permutation(n, a, c)


def library_init_model(seed, dim, vocab):
    """modelmats(0) as w2v_init_model fills it: (u - 0.5) / dim."""
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    n = dim * vocab
    blk = np.arange((n + 3) // 4, dtype=np.uint64)
    r = philox4x32_10((blk & np.uint64(0xFFFFFFFF)).astype(np.uint32),
                      (blk >> np.uint64(32)).astype(np.uint32), STREAM_INIT, 0, k0, k1)
    u = np.stack([u01(x) for x in r], axis=1).ravel()[:n]
    return ((u - np.float32(0.5)) / np.float32(dim)).astype(np.float32).reshape(vocab, dim)


# ---------------------------------------------------------------------------
# dobatch / evalbatch / Learner schedule on the CPU
# ---------------------------------------------------------------------------

def lrate_at(lrate0, texp, pos, first_pos):
    """lrate * (pos/firstPos)^(-texp)  (networks/Word2Vec.scala:170-173)."""
    nsteps = np.float32(np.float32(pos) / np.float32(first_pos))
    return np.float32(np.float32(lrate0) * np.float32(math.pow(float(nsteps), -float(np.float32(texp)))))


def eval_score(epos, eneg, nneg, ngoodwords, eq_pos_neg=False):
    """(epos + eneg / nneg) / goodwords.length  (networks/Word2Vec.scala:209)."""
    return (epos + eneg / (1 if eq_pos_neg else nneg)) / ngoodwords if ngoodwords else 0.0


def is_eval_step(istep, eval_step, has_next):
    """Learner.nextPass (Learner.scala:194): Scala's % keeps the dividend's sign,
    so istep 0 trains; istep 1, 1+evalStep, ... and the last batch only score."""
    rem = int(math.fmod(istep - 1, eval_step))
    return rem == 0 or (istep > 0 and not has_next)


class CpuWord2Vec:
    """The reference's CPU path driven minibatch by minibatch, with the uniform
    draws supplied by the caller: wordMats -> getnegs -> Pos -> Neg
    (networks/Word2Vec.scala:167-212, CPU branch)."""

    def __init__(self, opts, A, B, nthreads=1, impl="port"):
        self.o = dict(opts)
        self.A, self.B = A, B
        self.nthreads, self.impl = nthreads, impl
        self.first_pos = -1
        self.expt = expt_of(self.o["wexpt"])
        self.salpha = salpha_of(self.o["wsample"], self.o["vocabSize"])

    def wordmats(self, tokens, u_sample, u_window, prand, randneg):
        o = self.o
        words, lb, ub = wordmats_bounds(tokens, o["vocabSize"], o["nskip"], self.salpha, u_sample,
                                        u_window, o.get("iflip", False))
        WA, WB = getnegs(words, lb, ub, o["nneg"], o["nreuse"], o["vocabSize"], self.expt, prand,
                         randneg)
        return words, lb, ub, WA, WB

    def dobatch(self, tokens, pos, u_sample, u_window, prand, randneg):
        o = self.o
        if self.first_pos < 0:
            self.first_pos = pos
        lrpos = lrate_at(o["lrate"], o["texp"], pos, self.first_pos)
        lrneg = lrpos if o.get("eqPosNeg") else np.float32(lrpos / np.float32(o["nneg"]))
        words, lb, ub, WA, WB = self.wordmats(tokens, u_sample, u_window, prand, randneg)
        n = len(words)
        word2vecPos(o["dim"], n, o["nskip"], words, lb, ub, self.A, self.B, lrpos, o["vexp"],
                    self.nthreads, self.impl)
        word2vecNeg(o["dim"], WA.shape[0], o["nneg"], o["nreuse"], WA, WB, self.A, self.B, lrneg,
                    o["vexp"], self.nthreads, self.impl)
        return WB.size

    def evalbatch(self, tokens, u_sample, u_window, prand, randneg):
        o = self.o
        words, lb, ub, WA, WB = self.wordmats(tokens, u_sample, u_window, prand, randneg)
        epos = word2vecEvalPos(o["dim"], len(words), o["nskip"], words, lb, ub, self.A, self.B,
                               self.nthreads)
        eneg = word2vecEvalNeg(o["dim"], WA.shape[0], o["nneg"], o["nreuse"], WA, WB, self.A,
                               self.B, self.nthreads)
        return eval_score(epos, eneg, o["nneg"], WB.size, o.get("eqPosNeg", False))


def _draws(rng, n, nskip, nneg, nreuse):
    """Uniform draws one CPU minibatch consumes (numpy generator; the reference
    takes them from BIDMat's RNG, whose stream is not part of the checkout)."""
    cap = 2 * nskip * n
    return (rng.random(n, dtype=np.float32), rng.random(n, dtype=np.float32), rng.random(cap),
            rng.random(cap // nreuse * nneg + nneg, dtype=np.float32))


def cpu_learner_train(tokens, opts, batch_size, A, B, npasses=1, eval_step=11, seed=0, nthreads=1,
                      impl="port"):
    """Learner.nextPass (Learner.scala:173-252) driving the CPU model: returns the
    eval-step scores.  Short last minibatches are handed over and skipped by the
    model, as in the reference (networks/Word2Vec.scala:169,194)."""
    model = CpuWord2Vec(opts, A, B, nthreads, impl)
    rng = np.random.default_rng(seed)
    o = model.o
    here, scores = 0, []
    nb = -(-tokens.shape[0] // batch_size)
    for _ in range(npasses):
        for istep in range(nb):
            mb = tokens[istep * batch_size:(istep + 1) * batch_size]
            here += batch_size
            has_next = istep + 1 < nb
            if mb.shape[0] != batch_size:
                continue
            d = _draws(rng, batch_size, o["nskip"], o["nneg"], o["nreuse"])
            if is_eval_step(istep, eval_step, has_next):
                scores.append(model.evalbatch(mb, *d))
            else:
                model.dobatch(mb, here, *d)
    return scores


def cpu_learner_predict(tokens, opts, batch_size, A, B, seed=1, nthreads=1):
    """Learner.predict (Learner.scala:322-391): score of every full minibatch."""
    model = CpuWord2Vec(opts, A, B, nthreads, "port")
    rng = np.random.default_rng(seed)
    o = model.o
    out = []
    for k in range(tokens.shape[0] // batch_size):
        mb = tokens[k * batch_size:(k + 1) * batch_size]
        out.append(model.evalbatch(mb, *_draws(rng, batch_size, o["nskip"], o["nneg"], o["nreuse"])))
    return out
