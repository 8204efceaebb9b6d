"""Model export / import in the Google word2vec file format, as
``Word2Vec.saveGoogleW2V`` / ``readGoogleW2V`` write and read it
(src/main/scala/BIDMach/networks/Word2Vec.scala:1332-1394).

Layout: a text header ``"<nwords> <dim>\\n"``; then per word its string, a
space, the ``dim`` values and a newline.  In text mode each value is printed
with Java's ``%g`` followed by a space; in binary mode each value is the 4
bytes ``DataOutputStream.writeFloat`` emits, i.e. **big-endian** IEEE-754 (the
original C tool writes little-endian; files are therefore interchangeable with
it only in text mode).  The exported matrix is ``modelmats(0)``
(scripts/testword2vec.ssc:40).
"""
from __future__ import annotations

import io
import math

import numpy as np


def java_g(x: float) -> str:
    """``"%g" format x`` as java.util.Formatter prints a float: 6 significant
    digits, fixed notation for 1e-4 <= |x| < 1e6 (after rounding), scientific
    otherwise, trailing zeros kept."""
    x = float(x)
    if math.isnan(x):
        return "NaN"
    if math.isinf(x):
        return "Infinity" if x > 0 else "-Infinity"
    if x == 0.0:
        return "0.00000" if math.copysign(1.0, x) > 0 else "-0.00000"
    sci = "%.5e" % x                       # rounds to 6 significant digits
    exp = int(sci.split("e")[1])
    if -4 <= exp < 6:
        return "%.*f" % (5 - exp, x)
    mant, e = sci.split("e")
    return "%se%s%02d" % (mant, "-" if int(e) < 0 else "+", abs(int(e)))


def saveGoogleW2V(dict_words, mod, fname, binary: bool = False) -> int:
    """Writes ``mod`` (``[nwords_model, dim]``: one word vector per row, a numpy
    array or a CPU/CUDA tensor) with the words of ``dict_words`` (id order).  As
    the reference, only ``min(model words, dictionary length)`` words are
    written and a warning is printed when the dictionary is the shorter one.
    Returns the number of words written."""
    if hasattr(mod, "detach"):
        mod = mod.detach().cpu().numpy()
    mod = np.asarray(mod, dtype=np.float32)
    nmodel, dim = mod.shape
    if nmodel < len(dict_words):
        nwords = nmodel
    else:
        print("Warning: dictionary is smaller than model word count - you should reduce vocabSize "
              "in the Word2Vec model")
        nwords = len(dict_words)
    with open(fname, "wb") as f:
        f.write(("%d %d\n" % (nwords, dim)).encode())
        for i in range(nwords):
            f.write(dict_words[i].encode("utf-8") + b" ")
            if binary:
                f.write(mod[i].astype(">f4").tobytes())
            else:
                f.write("".join(java_g(v) + " " for v in mod[i]).encode())
            f.write(b"\n")
    return nwords


def readGoogleW2V(fname, dict_index, n: int, binary: bool = False) -> np.ndarray:
    """Reads a file written by ``saveGoogleW2V`` (or by the reference) into a
    ``[n, dim]`` float32 matrix; ``dict_index`` maps a word to its id (a dict or
    any callable returning -1 for unknown words); words with an id outside
    ``[0, n)`` are skipped, as in the reference."""
    lookup = dict_index if callable(dict_index) else (lambda w: dict_index.get(w, -1))
    with open(fname, "rb") as f:
        data = f.read()
    end = data.index(b"\n")
    nr, dim = (int(x) for x in data[:end].split())
    pos = end + 1
    model = np.zeros((n, dim), np.float32)
    for _ in range(nr):
        sp = data.index(b" ", pos)
        word = data[pos:sp].decode("utf-8")
        pos = sp + 1
        if binary:
            vec = np.frombuffer(data, dtype=">f4", count=dim, offset=pos).astype(np.float32)
            pos += 4 * dim
        else:
            nl = data.index(b"\n", pos)
            vec = np.array(data[pos:nl].split(), dtype=np.float32)
            if vec.size != dim:
                raise ValueError(f"word {word!r}: expected {dim} values, found {vec.size}")
            pos = nl
        if data[pos:pos + 1] == b"\n":
            pos += 1
        icol = lookup(word)
        if 0 <= icol < n:
            model[icol] = vec
    return model


# ---------------------------------------------------------------------------
# BIDMach checkpoint directory, Model.save / Model.load
# (src/main/scala/BIDMach/models/Model.scala:245-315): ``<fname>options.json``
# and one ``<fname>modelmat%02d.lz4`` per model matrix (BIDMat matrix file,
# dim x vocab column-major, which is the [vocab, dim] row-major buffer of this
# package).  ``fname`` normally ends in "/" (a directory, created if needed);
# otherwise it is a prefix, as in the reference.  The reference also writes
# ``options.ser`` (Java serialisation of the options object), which has no
# meaning outside a JVM: it is not written, and ``load`` is the reference's
# ``load(fname, useJson = true)``.
# ---------------------------------------------------------------------------
def saveModel(fname: str, opts: dict, mats) -> None:
    import json
    import os

    from . import matio
    parent = os.path.dirname(fname + "options.json")
    if parent:
        os.makedirs(parent, exist_ok=True)
    with open(fname + "options.json", "w") as f:
        json.dump(opts, f, indent=1, sort_keys=True)
    for i, m in enumerate(mats):
        if hasattr(m, "detach"):
            m = m.detach().cpu().numpy()
        matio.saveMat(fname + "modelmat%02d.lz4" % i, np.asarray(m).T)


def loadModel(fname: str):
    """Returns ``(opts dict, [matrix, ...])``; each matrix comes back as
    ``[vocab, dim]`` (a view of the file's bytes, read-only)."""
    import json
    import os

    from . import matio
    with open(fname + "options.json") as f:
        opts = json.load(f)
    mats, n = [], 0
    while os.path.exists(fname + "modelmat%02d.lz4" % n):
        mats.append(matio.loadMat(fname + "modelmat%02d.lz4" % n).T)
        n += 1
    return opts, mats


def deleteModel(fname: str) -> None:
    """Model.delete (models/Model.scala:266-280): the files ``saveModel`` wrote, then the
    directory if that leaves it empty."""
    import os
    names = [fname + "options.json", fname + "options.ser"]
    n = 0
    while os.path.exists(fname + "modelmat%02d.lz4" % n):
        names.append(fname + "modelmat%02d.lz4" % n)
        n += 1
    for f in names:
        if os.path.exists(f):
            os.remove(f)
    parent = os.path.dirname(fname + "options.json")
    if parent and os.path.isdir(parent) and not os.listdir(parent):
        os.rmdir(parent)
