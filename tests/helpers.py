"""Input builders shared by the CPU and GPU tests."""
from __future__ import annotations

import numpy as np


def random_model(vocab, dim, seed, scale=None):
    rng = np.random.default_rng(seed)
    scale = scale if scale is not None else 1.0 / dim
    A = ((rng.random((vocab, dim), dtype=np.float32) - 0.5) * np.float32(2 * scale)).astype(np.float32)
    B = ((rng.random((vocab, dim), dtype=np.float32) - 0.5) * np.float32(2 * scale)).astype(np.float32)
    return A, B


def conflict_free_pos(ncols, vocab, skip, seed, drop=0.1):
    """Positive-pair inputs on which the sequential CPU update and a parallel
    update agree: all word ids distinct, and full windows only at centres spaced
    2*skip+1 apart so that every context position belongs to one centre."""
    assert ncols <= vocab
    rng = np.random.default_rng(seed)
    W = rng.permutation(vocab)[:ncols].astype(np.int32)
    W[rng.random(ncols) < drop] = -1
    LB = np.zeros(ncols, np.int32)
    UB = np.zeros(ncols, np.int32)
    centres = np.arange(skip, ncols, 2 * skip + 1)
    lo = rng.integers(1, skip + 1, size=len(centres))
    LB[centres] = -np.minimum(lo, centres)
    UB[centres] = np.minimum(lo, ncols - 1 - centres)
    return W, LB, UB


def conflict_free_neg(ncols, vocab, nwa, nwb, seed):
    """All ids of WA distinct and all ids of WB distinct over the whole input."""
    assert ncols * max(nwa, nwb) <= vocab
    rng = np.random.default_rng(seed)
    WA = rng.permutation(vocab)[: ncols * nwa].astype(np.int32).reshape(ncols, nwa)
    WB = rng.permutation(vocab)[: ncols * nwb].astype(np.int32).reshape(ncols, nwb)
    return WA, WB


def random_pos(ncols, vocab, skip, seed, drop=0.15, doc_len=37):
    """General (conflicting) positive-pair inputs with sentence-clipped windows."""
    rng = np.random.default_rng(seed)
    W = rng.integers(0, vocab, size=ncols).astype(np.int32)
    W[rng.random(ncols) < drop] = -1
    pos_in_doc = np.arange(ncols) % doc_len
    left = np.minimum(pos_in_doc, ncols)
    right = np.minimum(doc_len - 1 - pos_in_doc, ncols - 1 - np.arange(ncols))
    r = rng.integers(1, skip + 1, size=ncols)
    LB = -np.minimum(r, left).astype(np.int32)
    UB = np.minimum(r, right).astype(np.int32)
    return W, LB, UB


def random_neg(ncols, vocab, nwa, nwb, seed):
    rng = np.random.default_rng(seed)
    WA = rng.integers(0, vocab, size=(ncols, nwa)).astype(np.int32)
    WB = rng.integers(0, vocab, size=(ncols, nwb)).astype(np.int32)
    return WA, WB


def rel_err(got, want):
    """max |got - want| / max |want| : the "relative" of the 1e-5 kernel bar."""
    denom = float(np.max(np.abs(want)))
    return float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64)))) / (denom or 1.0)


def elem_rel_err(got, want, floor_frac=0.01):
    """Element-wise companion of rel_err: max over elements of |got - want| / max(|want|, floor),
    floor = floor_frac * max |want|.  An element far below the floor is a sum of terms that nearly
    cancel; its fp32 rounding error follows the terms, not the sum, so it is measured against the
    floor instead.  The kernels are held to 1e-4 here (1e-5 norm-wise in rel_err)."""
    want = want.astype(np.float64)
    floor = floor_frac * float(np.max(np.abs(want))) or 1.0
    return float(np.max(np.abs(got.astype(np.float64) - want) / np.maximum(np.abs(want), floor)))
