"""Every tutorial script runs to the end (reduced sizes, CPU)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CASES = [
    ("building_image_classifier.py", ["--samples", "256", "--epochs", "1", "--device", "cpu"], "test accuracy"),
    ("building_lstm_name_classifier.py", ["--samples", "400", "--epochs", "1", "--device", "cpu"], "test accuracy"),
    ("building_text_classifier.py", ["--samples", "400", "--epochs", "1", "--device", "cpu"], "test accuracy"),
    ("guide_to_grad_sampler.py", [], "per-sample gradients match the micro-batch oracle"),
    ("guide_to_module_validator.py", [], "SampleMaxScale"),
    ("intro_to_advanced_features.py", [], "4 accounted steps"),
    ("non_wrapping_mode.py", [], "after remove_hooks"),
    ("ddp_tutorial.py", ["--spawn", "2", "--cpu", "--epochs", "1", "--port", "29541"], "replicas identical: True"),
]


@pytest.mark.parametrize("script,argv,expect", CASES, ids=[c[0] for c in CASES])
def test_tutorial_runs(script, argv, expect):
    env = dict(os.environ, PYTHONWARNINGS="ignore", CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "tutorials", script), *argv], capture_output=True, text=True,
                         timeout=600, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    assert expect in out.stdout, out.stdout[-2000:]


def test_notebooks_match_their_scripts():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "tutorials", "make_notebooks.py"), "--check"],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr


def test_a_notebook_executes_cell_by_cell():
    """The code cells of one generated notebook run in order in a fresh namespace, from the notebooks folder."""
    import json

    path = os.path.join(ROOT, "tutorials", "notebooks", "guide_to_module_validator.ipynb")
    with open(path, encoding="utf-8") as f:
        cells = [c for c in json.load(f)["cells"] if c["cell_type"] == "code"]
    program = "\n\n".join("".join(c["source"]) for c in cells)
    out = subprocess.run([sys.executable, "-c", program], capture_output=True, text=True, timeout=300,
                         cwd=os.path.join(ROOT, "tutorials", "notebooks"),
                         env=dict(os.environ, PYTHONWARNINGS="ignore", CUDA_VISIBLE_DEVICES=""))
    assert out.returncode == 0, out.stderr[-2000:]
    assert "SampleMaxScale" in out.stdout
