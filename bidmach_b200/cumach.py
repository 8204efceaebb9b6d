"""Python face of ``edu.berkeley.bid.CUMACH`` for the Word2Vec path.

Same method names, argument order and return convention as the Java class
(src/main/java/edu/berkeley/bid/CUMACH.java:90-98): every method returns an int,
0 on success, otherwise a CUDA error code (or 1 for an unsupported shape).  The
``Pointer`` arguments of the Java methods are device buffers here: anything with
a ``data_ptr()`` (a CUDA ``torch.Tensor``) or a plain integer address.

The calls go straight to the C-ABI library; there is no other implementation.
"""
from __future__ import annotations

from . import _lib


def _addr(x) -> int:
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    if hasattr(x, "is_cuda"):
        if not x.is_cuda:
            raise ValueError("CUMACH expects device buffers (CUDA tensors)")
        if not x.is_contiguous():
            raise ValueError("CUMACH expects contiguous buffers")
    return int(x.data_ptr())


class CUMACH:
    """Static methods only, like the Java class."""

    @staticmethod
    def word2vecPos(nrows, ncols, shift, W, LB, UB, A, B, lrate, vexp) -> int:
        return _lib.load().word2vecPos(nrows, ncols, shift, _addr(W), _addr(LB), _addr(UB),
                                       _addr(A), _addr(B), lrate, vexp)

    @staticmethod
    def word2vecNeg(nrows, ncols, nwa, nwb, WA, WB, A, B, lrate, vexp) -> int:
        return _lib.load().word2vecNeg(nrows, ncols, nwa, nwb, _addr(WA), _addr(WB), _addr(A),
                                       _addr(B), lrate, vexp)

    @staticmethod
    def word2vecNegFilt(nrows, ncols, nwords, nwa, nwb, WA, WB, A, B, lrate, vexp) -> int:
        return _lib.load().word2vecNegFilt(nrows, ncols, nwords, nwa, nwb, _addr(WA), _addr(WB),
                                           _addr(A), _addr(B), lrate, vexp)

    @staticmethod
    def word2vecEvalPos(nrows, ncols, shift, W, LB, UB, A, B, retVal) -> int:
        return _lib.load().word2vecEvalPos(nrows, ncols, shift, _addr(W), _addr(LB), _addr(UB),
                                           _addr(A), _addr(B), _addr(retVal))

    @staticmethod
    def word2vecEvalNeg(nrows, ncols, nwa, nwb, WA, WB, A, B, retVal) -> int:
        return _lib.load().word2vecEvalNeg(nrows, ncols, nwa, nwb, _addr(WA), _addr(WB), _addr(A),
                                           _addr(B), _addr(retVal))


class CUMACHSlice:
    """Device forms of ``CPUMACH.word2vecPosSlice`` / ``word2vecNegSlice``
    (src/main/java/edu/berkeley/bid/CPUMACH.java) and of the Scala scoring twins
    ``Word2Vec.evalPosCPUslice`` / ``evalNegCPUslice``: one vocabulary slice per call, its rows in
    one matrix per side (no ``maxCols`` blocks, no ``dualMode``)."""

    @staticmethod
    def word2vecPosSlice(nrows, ncols, shift, W, LB, UB, A, B, lrate, vexp, islice, nslices, nHead, doHead=1) -> int:
        return _lib.load().word2vecPosSlice(nrows, ncols, shift, _addr(W), _addr(LB), _addr(UB), _addr(A),
                                            _addr(B), lrate, vexp, islice, nslices, nHead, doHead)

    @staticmethod
    def word2vecNegSlice(nrows, ncols, nwa, nwb, WA, WB, A, B, lrate, vexp, islice, nslices, nHead, doHead=1) -> int:
        return _lib.load().word2vecNegSlice(nrows, ncols, nwa, nwb, _addr(WA), _addr(WB), _addr(A), _addr(B),
                                            lrate, vexp, islice, nslices, nHead, doHead)

    @staticmethod
    def word2vecEvalPosSlice(nrows, ncols, shift, W, LB, UB, A, B, retVal, islice, nslices, nHead) -> int:
        return _lib.load().word2vecEvalPosSlice(nrows, ncols, shift, _addr(W), _addr(LB), _addr(UB), _addr(A),
                                                _addr(B), _addr(retVal), islice, nslices, nHead)

    @staticmethod
    def word2vecEvalNegSlice(nrows, ncols, nwa, nwb, WA, WB, A, B, retVal, islice, nslices, nHead) -> int:
        return _lib.load().word2vecEvalNegSlice(nrows, ncols, nwa, nwb, _addr(WA), _addr(WB), _addr(A),
                                                _addr(B), _addr(retVal), islice, nslices, nHead)


def word2vecEvalNegNoAlloc(nrows, ncols, nwa, nwb, WA, WB, A, B, retVal) -> int:
    """``CUMACH.word2vecEvalNeg`` for callers that cannot allocate device memory
    while running (the Java class has no such method).  Same arguments and
    result; its scratch memory is an array inside the library, so it accepts at
    most 2,097,152 columns per call, returns 1 beyond that, and must not run
    concurrently with another call of itself on the same GPU."""
    return _lib.load().word2vecEvalNegNoAlloc(nrows, ncols, nwa, nwb, _addr(WA), _addr(WB),
                                              _addr(A), _addr(B), _addr(retVal))


def cuda_error_string(err: int) -> str:
    """Text for a code returned by the methods above (cudaGetErrorString)."""
    if err == 0:
        return "no error"
    try:
        import torch
        return f"CUDA error {err}: " + torch.cuda.cudart().cudaGetErrorString(err)  # type: ignore[attr-defined]
    except Exception:
        return f"CUDA error {err}"
