"""Generates the golden fixtures of this directory from the reference's own CPU
kernels (jni/src/BIDMach_CPUMACH.c compiled unchanged, oracle/_ref/libw2vref.so).

Run once on a machine that has the BIDMach checkout:

    python tests/golden/make_golden.py

Each kernels_*.npz holds seeded inputs and the model matrices after the
reference's word2vecPos, then after its word2vecNeg (nthreads = 1, so the
result is deterministic); each slices_*.npz the same for word2vecPosSlice and
word2vecNegSlice on one vocabulary slice.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from helpers import random_model, random_neg, random_pos  # noqa: E402
from oracle import oracle as orc  # noqa: E402

CASES = [  # dim, vocab, skip, ncols, nwa, nwb, ngroups, seed
    (100, 120, 5, 96, 5, 5, 40, 1),
    (300, 60, 5, 64, 5, 5, 24, 2),
    (300, 60, 3, 48, 10, 5, 12, 3),
    (64, 80, 2, 80, 5, 10, 16, 4),
    (100, 50, 5, 50, 5, 1, 30, 5),
]


SLICE_CASES = [  # dim, vocab, skip, ncols, nwa, nwb, ngroups, nslices, islice, nhead, do_head, seed
    (64, 160, 5, 96, 5, 5, 30, 4, 1, 12, 1, 11),
    (100, 120, 3, 80, 10, 5, 16, 2, 1, 30, 0, 12),
    (64, 200, 5, 96, 5, 5, 30, 8, 5, 16, 2, 13),
]


def slices():
    """slices_*.npz: the reference's word2vecPosSlice, then its word2vecNegSlice, on one slice's
    matrices (a single block of maxCols words per side)."""
    for dim, vocab, skip, ncols, nwa, nwb, ng, nslices, islice, nhead, do_head, seed in SLICE_CASES:
        rows = orc.slice_rows(vocab, nslices, nhead)
        A, B = random_model(rows, dim, seed, scale=0.5)
        W, LB, UB = random_pos(ncols, vocab, skip, seed)
        WA, WB = random_neg(ng, vocab, nwa, nwb, seed + 100)
        lrate, vexp = np.float32(0.05), np.float32(0.5)
        A1, B1 = A.copy(), B.copy()
        orc.word2vecPosSlice(dim, ncols, skip, W, LB, UB, A1, B1, lrate, vexp, islice, nslices, nhead, do_head, 1,
                             "reference")
        A2, B2 = A1.copy(), B1.copy()
        orc.word2vecNegSlice(dim, ng, nwa, nwb, WA, WB, A2, B2, float(lrate) / nwa, vexp, islice, nslices, nhead,
                             do_head, 1, "reference")
        np.savez_compressed(os.path.join(HERE, f"slices_n{nslices}_i{islice}_h{nhead}_d{do_head}.npz"),
                            dim=dim, skip=skip, lrate=lrate, vexp=vexp, nslices=nslices, islice=islice, nhead=nhead,
                            do_head=do_head, W=W, LB=LB, UB=UB, WA=WA, WB=WB, A=A, B=B, A_pos=A1, B_pos=B1,
                            A_neg=A2, B_neg=B2)
        print("wrote slice", nslices, islice, nhead, do_head)


def main():
    assert orc.have_reference(), "needs the compiled reference"
    slices()
    for dim, vocab, skip, ncols, nwa, nwb, ng, seed in CASES:
        A, B = random_model(vocab, dim, seed, scale=0.5)
        W, LB, UB = random_pos(ncols, vocab, skip, seed)
        WA, WB = random_neg(ng, vocab, nwa, nwb, seed + 100)
        lrate, vexp = np.float32(0.05), np.float32(0.5)
        A1, B1 = A.copy(), B.copy()
        orc.word2vecPos(dim, ncols, skip, W, LB, UB, A1, B1, lrate, vexp, 1, "reference")
        A2, B2 = A1.copy(), B1.copy()
        orc.word2vecNeg(dim, ng, nwa, nwb, WA, WB, A2, B2, float(lrate) / nwa, vexp, 1, "reference")
        np.savez_compressed(os.path.join(HERE, f"kernels_d{dim}_s{skip}_{nwa}x{nwb}.npz"),
                            dim=dim, skip=skip, lrate=lrate, vexp=vexp, W=W, LB=LB, UB=UB, WA=WA,
                            WB=WB, A=A, B=B, A_pos=A1, B_pos=B1, A_neg=A2, B_neg=B2)
        print("wrote", dim, skip, nwa, nwb)


if __name__ == "__main__":
    main()
