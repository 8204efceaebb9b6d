"""Loader of the C-ABI library ``libbidmachcuda-linux-x86_64.so``.

There is no fallback: if the library is missing or cannot be loaded, importing
anything that computes raises, naming the build command.
"""
from __future__ import annotations

import ctypes as C
import os

LIB_NAME = "libbidmachcuda-linux-x86_64.so"
LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), LIB_NAME)

_I = C.c_int
_F = C.c_float
_P = C.c_void_p


class W2VOpts(C.Structure):
    """``w2v_opts`` of include/bidmach_b200.h."""
    _fields_ = [("dim", _I), ("nskip", _I), ("nneg", _I), ("nreuse", _I), ("vocabSize", _I),
                ("wexpt", _F), ("wsample", _F), ("lrate", _F), ("texp", _F), ("vexp", _F),
                ("iflip", _I), ("eqPosNeg", _I), ("permute", _I), ("seed", C.c_uint64)]


class W2VUniforms(C.Structure):
    """``w2v_uniforms``: optional device arrays of explicit uniform draws."""
    _fields_ = [("sample", _P), ("window", _P), ("permute", _P), ("negs", _P)]


class W2VBuffers(C.Structure):
    """``w2v_buffers_t``: device addresses of the latest preprocessing results."""
    _fields_ = [("words", _P), ("lb", _P), ("ub", _P), ("contexts", _P), ("WB", _P), ("WA", _P),
                ("npairs", C.c_int64), ("ngroups", _I)]


class W2VTiming(C.Structure):
    """``w2v_timing``: summed phase durations (ms) and work counts."""
    _fields_ = [("prep_ms", C.c_double), ("permute_ms", C.c_double), ("pos_ms", C.c_double),
                ("neg_ms", C.c_double), ("evalpos_ms", C.c_double), ("evalneg_ms", C.c_double),
                ("train_batches", C.c_int64), ("eval_batches", C.c_int64), ("pairs", C.c_int64),
                ("groups", C.c_int64), ("eval_pairs", C.c_int64), ("eval_groups", C.c_int64)]


# name -> (restype, argtypes); every symbol include/bidmach_b200.h declares
SIGNATURES = {
    "word2vecPos": (_I, [_I, _I, _I, _P, _P, _P, _P, _P, _F, _F]),
    "word2vecNeg": (_I, [_I, _I, _I, _I, _P, _P, _P, _P, _F, _F]),
    "word2vecNegFilt": (_I, [_I, _I, _I, _I, _I, _P, _P, _P, _P, _F, _F]),
    "word2vecEvalPos": (_I, [_I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "word2vecEvalNeg": (_I, [_I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "word2vecPosSlice": (_I, [_I, _I, _I, _P, _P, _P, _P, _P, _F, _F, _I, _I, _I, _I]),
    "word2vecNegSlice": (_I, [_I, _I, _I, _I, _P, _P, _P, _P, _F, _F, _I, _I, _I, _I]),
    "word2vecEvalPosSlice": (_I, [_I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I]),
    "word2vecEvalNegSlice": (_I, [_I, _I, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I]),
    "word2vecEvalNegNoAlloc": (_I, [_I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "bidmach_xxh32": (C.c_uint32, [_P, C.c_int64, C.c_uint32]),
    "bidmach_lz4_compress_bound": (C.c_int64, [C.c_int64]),
    "bidmach_lz4_compress": (C.c_int64, [_P, C.c_int64, _P, C.c_int64]),
    "bidmach_lz4_decompress": (C.c_int64, [_P, C.c_int64, _P, C.c_int64]),
    "JNI_OnLoad": (_I, [_P, _P]),
    "Java_edu_berkeley_bid_CUMACH_word2vecPos": (_I, [_P, _P, _I, _I, _I, _P, _P, _P, _P, _P, _F, _F]),
    "Java_edu_berkeley_bid_CUMACH_word2vecNeg": (_I, [_P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _F, _F]),
    "Java_edu_berkeley_bid_CUMACH_word2vecNegFilt": (_I, [_P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _F, _F]),
    "Java_edu_berkeley_bid_CUMACH_word2vecEvalPos": (_I, [_P, _P, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "Java_edu_berkeley_bid_CUMACH_word2vecEvalNeg": (_I, [_P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "Java_edu_berkeley_bid_CUMACH_w2vCreate": (C.c_int64, [_P, _P, _I, _I, _I, _I, _I, _F, _F, _F, _F, _F, _I, _I, _I,
                                                           C.c_int64, _I]),
    "Java_edu_berkeley_bid_CUMACH_w2vDestroy": (None, [_P, _P, C.c_int64]),
    "Java_edu_berkeley_bid_CUMACH_w2vInitModel": (_I, [_P, _P, C.c_int64, _P, _P]),
    "Java_edu_berkeley_bid_CUMACH_w2vDobatch": (_I, [_P, _P, C.c_int64, _P, _P, _P, C.c_int64, C.c_int64]),
    "Java_edu_berkeley_bid_CUMACH_w2vEvalbatch": (C.c_double, [_P, _P, C.c_int64, _P, _P, _P, C.c_int64]),
    "Java_edu_berkeley_bid_CUMACH_w2vLastError": (_I, [_P, _P, C.c_int64]),
    "Java_edu_berkeley_bid_CUMACH_w2vSetSlice": (_I, [_P, _P, C.c_int64, _I, _I, _I, _I]),
    "Java_edu_berkeley_bid_CUMACH_word2vecPosSlice": (_I, [_P, _P, _I, _I, _I, _P, _P, _P, _P, _P, _F, _F, _I, _I, _I, _I]),
    "Java_edu_berkeley_bid_CUMACH_word2vecNegSlice": (_I, [_P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _F, _F, _I, _I, _I, _I]),
    "Java_edu_berkeley_bid_CUMACH_word2vecEvalPosSlice": (_I, [_P, _P, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I]),
    "Java_edu_berkeley_bid_CUMACH_word2vecEvalNegSlice": (_I, [_P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I]),
    "Java_edu_berkeley_bid_CUMACH_w2vCommInitAll": (C.c_int64, [_P, _P, _I]),
    "Java_edu_berkeley_bid_CUMACH_w2vCommOf": (C.c_int64, [_P, _P, C.c_int64, _I]),
    "Java_edu_berkeley_bid_CUMACH_w2vAllreduceAvg": (_I, [_P, _P, C.c_int64, _P, _P, C.c_int64]),
    "Java_edu_berkeley_bid_CUMACH_w2vCommDestroyAll": (None, [_P, _P, C.c_int64]),
    "w2v_default_opts": (None, [C.POINTER(W2VOpts)]),
    "w2v_create": (_I, [C.POINTER(W2VOpts), _I, C.POINTER(_P)]),
    "w2v_destroy": (None, [_P]),
    "w2v_init_model": (_I, [C.POINTER(W2VOpts), _P, _P, _P]),
    "w2v_wordmats": (_I, [_P, _P, C.POINTER(W2VUniforms), C.c_uint64, _P]),
    "w2v_buffers": (_I, [_P, C.POINTER(W2VBuffers)]),
    "w2v_dobatch": (_I, [_P, _P, C.POINTER(W2VUniforms), _P, _P, C.c_int64, C.c_uint64, _P]),
    "w2v_evalbatch": (_I, [_P, _P, C.POINTER(W2VUniforms), _P, _P, C.c_uint64, C.POINTER(C.c_double), _P]),
    "w2v_dobatch_host": (_I, [_P, _P, _P, _P, C.c_int64, C.c_uint64, C.POINTER(C.c_int64), _P]),
    "w2v_evalbatch_host": (_I, [_P, _P, _P, _P, C.c_uint64, C.POINTER(C.c_double), _P]),
    "w2v_apply_average": (_I, [_P, _P, _P, C.c_int64, _P]),
    "w2v_comm_init_all": (_I, [_I, C.POINTER(_I), C.POINTER(_P)]),
    "w2v_comm_unique_id": (_I, [_P]),
    "w2v_comm_init_rank": (_I, [_I, _I, _P, C.POINTER(_P)]),
    "w2v_comm_register": (_I, [_P, _P, C.c_int64]),
    "w2v_allreduce_avg": (_I, [_P, _P, _P, C.c_int64, _P]),
    "w2v_comm_destroy": (None, [_P]),
    "w2v_nvls_average": (_I, [_P, C.c_int64, _I, _I, _I, _P]),
    "w2v_p2p_average": (_I, [C.POINTER(_P), C.c_int64, _I, _I, _I, _P]),
    "w2v_wait_pos": (_I, [_P, _P]),
    "w2v_wait_before_neg": (_I, [_P, _P]),
    "w2v_reserve_sms": (_I, [_P, _I]),
    "w2v_set_slice": (_I, [_P, _I, _I, _I, _I]),
    "w2v_slice_rows": (C.c_int64, [_I, _I, _I]),
    "w2v_set_timing": (_I, [_P, _I]),
    "w2v_get_timing": (_I, [_P, C.POINTER(W2VTiming)]),
    "w2v_launch_count": (C.c_longlong, []),
}

_lib = None


def load() -> C.CDLL:
    """Loads the library once and types its entry points."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_NAME} is not built: run `python -m bidmach_b200.csrc.build` "
                "(needs nvcc; there is no CPU or PyTorch fallback for this path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
