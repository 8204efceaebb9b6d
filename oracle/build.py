"""Build recipe for the CPU oracle (test infrastructure, not product code).

Two shared objects:

* ``oracle/libw2v_oracle.so``  -- this repository's C restatement
  (``w2v_oracle.c``); always built.
* ``oracle/_ref/libw2vref.so`` -- the reference's own CPU kernels, compiled
  from ``jni/src/BIDMach_CPUMACH.c`` where that file lies inside a BIDMach
  checkout (never copied here), plus ``ref_driver.c`` and the stand-in
  ``stub_jni/jni.h``.  Built only when the checkout is present; on a machine
  without it the previously built file is used as is.

Both use the same flags (``-O2 -fopenmp -ffp-contract=off``, no ``-march``) so
that the restatement and the reference round identically and can be compared
bit for bit.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# a BIDMach checkout: $BIDMACH_REFERENCE, else a directory "reference" beside this repository
REF_ROOT = os.environ.get("BIDMACH_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
REF_SRC = os.path.join(REF_ROOT, "jni", "src", "BIDMach_CPUMACH.c")

ORACLE_SO = os.path.join(HERE, "libw2v_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libw2vref.so")

CFLAGS = ["-O2", "-fopenmp", "-ffp-contract=off", "-fPIC", "-shared", "-fvisibility=hidden"]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "w2v_oracle.c")
    if force or not _newer(ORACLE_SO, [src]):
        subprocess.check_call(["gcc", *CFLAGS, src, "-o", ORACLE_SO, "-lm"])
    return ORACLE_SO


def build_ref(force: bool = False) -> str | None:
    """Compile the reference CPU kernels in place.  Returns None when neither
    the reference sources nor a previously built library are available."""
    if not os.path.exists(REF_SRC):
        return REF_SO if os.path.exists(REF_SO) else None
    drv = os.path.join(HERE, "ref_driver.c")
    stub = os.path.join(HERE, "stub_jni")
    if force or not _newer(REF_SO, [REF_SRC, drv, os.path.join(stub, "jni.h")]):
        os.makedirs(REF_DIR, exist_ok=True)
        # the reference is compiled with default symbol visibility (it has no
        # export annotations of its own beyond JNIEXPORT from the stub header)
        flags = [f for f in CFLAGS if f != "-fvisibility=hidden"]
        subprocess.check_call(["gcc", *flags, "-w", "-I", stub, REF_SRC, drv, "-o", REF_SO, "-lm"])
    return REF_SO


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_ref(force))
