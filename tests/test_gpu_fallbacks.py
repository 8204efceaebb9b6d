"""The kernels that only run when the preferred one does not fit (or is switched off
for an experiment) must pass the same parity tests: the register-resident negative
kernels (W2V_NEG_IMPL=reg) and plain atomics without hot-row replicas
(W2V_HOT_LEVELS=0).  The switches are read once per process, hence the subprocesses."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rerun(env_extra, keyword):
    env = dict(os.environ, **env_extra)
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join("tests", "test_gpu_kernels.py"), "-m", "gpu",
                        "-q", "-x", "-k", keyword, "-p", "no:cacheprovider"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-1000:]
    assert " passed" in r.stdout


def test_register_resident_negative_kernels_pass_the_parity_tests():
    _rerun({"W2V_NEG_IMPL": "reg"}, "neg or Neg")


def test_plain_atomics_without_hot_row_replicas_pass_the_parity_tests():
    _rerun({"W2V_HOT_LEVELS": "0"}, "neg or Neg or pos or Pos")
