"""Runs a fast subset of the reference library's own tests against this package
through the import alias in ``conformance_plugin.py``.  Skipped unless
``OPACUS_REFERENCE_TESTS`` points at a reference checkout's ``opacus/tests``."""
import os
import subprocess
import sys

import pytest

REF = os.environ.get("OPACUS_REFERENCE_TESTS", "")
SUBSET = ["accountants_test.py", "grad_samples/linear_test.py", "grad_samples/embedding_norm_sample_test.py",
          "schedulers", "validators", "batch_memory_manager_test.py", "module_validator_test.py",
          "grad_sample_module_test.py", "poisson_test.py"]


@pytest.mark.skipif(not os.path.isdir(REF), reason="OPACUS_REFERENCE_TESTS is not set")
def test_reference_suite_subset():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-p", "tests.conformance_plugin"] + \
          [os.path.join(REF, s) for s in SUBSET]
    res = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=3000)
    assert res.returncode == 0, res.stdout[-4000:]
