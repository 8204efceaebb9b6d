"""The C-ABI library loads without a GPU and exports every function that
include/bidmach_b200.h declares (no compute calls here)."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "bidmach_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"^\s*(?:int|void|long long|int64_t|uint32_t|double)\s+\**(\w+)\s*\(", text, flags=re.M)
    return sorted(set(names))


def test_header_declares_the_reference_entry_points():
    names = _declared_functions()
    for n in ["word2vecPos", "word2vecNeg", "word2vecNegFilt", "word2vecEvalPos", "word2vecEvalNeg",
              "JNI_OnLoad", "Java_edu_berkeley_bid_CUMACH_word2vecPos",
              "Java_edu_berkeley_bid_CUMACH_word2vecNeg", "Java_edu_berkeley_bid_CUMACH_word2vecNegFilt",
              "Java_edu_berkeley_bid_CUMACH_word2vecEvalPos", "Java_edu_berkeley_bid_CUMACH_word2vecEvalNeg"]:
        assert n in names


def test_library_exports_every_declared_symbol():
    from bidmach_b200 import _lib
    lib = C.CDLL(_lib.LIB_PATH)
    for n in _declared_functions():
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"


def test_python_signature_table_covers_the_header():
    from bidmach_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared_functions()
    _lib.load()


def test_library_name_follows_the_reference_loader():
    from bidmach_b200 import _lib
    assert os.path.basename(_lib.LIB_PATH) == "libbidmachcuda-linux-x86_64.so"


def test_default_opts_match_the_reference_defaults():
    from bidmach_b200 import _lib
    from bidmach_b200.word2vec import Opts
    o = _lib.W2VOpts()
    _lib.load().w2v_default_opts(C.byref(o))
    p = Opts()
    assert (o.dim, o.nskip, o.nneg, o.nreuse, o.vocabSize) == (256, 5, 5, 5, 100000)
    assert (o.dim, o.nskip, o.nneg, o.nreuse, o.vocabSize) == (p.dim, p.nskip, p.nneg, p.nreuse, p.vocabSize)
    assert abs(o.wexpt - 0.75) < 1e-7 and abs(o.wsample - 1e-4) < 1e-10
    assert (o.lrate, o.texp, o.vexp) == (1.0, 0.5, 0.5)


def test_product_code_never_touches_the_oracle():
    """Nothing under the package may import, load or execute the oracle."""
    pkg = os.path.join(ROOT, "bidmach_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "__none__", os.path.join(dirpath, f)
