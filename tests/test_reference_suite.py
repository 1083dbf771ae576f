"""The reference's own test files, unmodified, against this library under the reference's name.

Set ``RESKV_REFERENCE_CHECKOUT`` to a checkout of the reference (its ``tests/`` folder is all that is
read); without it these tests are skipped.  The files are run by a child pytest whose import path has
this repository first, so ``import reskv`` resolves to the alias package at the repository root and
through it to ``reskv_b200``.

``tests/test_config.py``: everything passes except the three cases that construct the reference's
accuracy-simulation models, which this library does not contain.  ``tests/test_cuda.py`` (needs the
GPU): every case passes.
"""

import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CHECKOUT = os.environ.get("RESKV_REFERENCE_CHECKOUT")
needs_checkout = pytest.mark.skipif(not CHECKOUT, reason="RESKV_REFERENCE_CHECKOUT is not set")

ACCURACY_ONLY = {
    "test_model_rejects_configuration_of_other_implementation[accuracy]",
    "test_model_rejects_configuration_of_other_architecture[llama_accuracy]",
    "test_model_rejects_configuration_of_other_architecture[qwen3_accuracy]",
}


def _run(test_file: str, tmp_path):
    env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "pytest", str(Path(CHECKOUT) / "tests" / test_file), "-q", "-p", "no:cacheprovider",
           "-rf", "--rootdir", str(tmp_path)]
    r = subprocess.run(cmd, cwd=tmp_path, env=env, capture_output=True, text=True, timeout=1800)
    failed = set(re.findall(r"^FAILED \S*::(\S+)", r.stdout, flags=re.M))
    counts = {k: int(v) for v, k in re.findall(r"(\d+) (passed|failed|skipped|error)", r.stdout.splitlines()[-1])}
    # the child must have used this repository's alias, not the checkout's package
    probe = subprocess.run([sys.executable, "-c", "import reskv; print(reskv.__file__)"], cwd=tmp_path, env=env,
                           capture_output=True, text=True)
    assert Path(probe.stdout.strip()).resolve() == (ROOT / "reskv" / "__init__.py").resolve(), probe.stdout + probe.stderr
    return counts, failed, r.stdout[-3000:]


@needs_checkout
def test_reference_config_tests(tmp_path):
    counts, failed, tail = _run("test_config.py", tmp_path)
    assert failed == ACCURACY_ONLY, tail
    assert counts.get("passed", 0) >= 70 and counts.get("error", 0) == 0, tail


@needs_checkout
def test_reference_mlp_tests(tmp_path):
    """``tests/test_mlp.py`` of the reference (equality with the stock MLP, gradients untouched); its one
    CUDA case is skipped on a machine without a GPU."""
    counts, failed, tail = _run("test_mlp.py", tmp_path)
    assert not failed and counts.get("error", 0) == 0 and counts.get("passed", 0) >= 3, tail


@needs_checkout
@pytest.mark.gpu
def test_reference_cuda_tests(tmp_path):
    counts, failed, tail = _run("test_cuda.py", tmp_path)
    assert not failed and counts.get("failed", 0) == 0 and counts.get("error", 0) == 0, tail
    assert counts.get("passed", 0) >= 33 and counts.get("skipped", 0) == 0, tail
