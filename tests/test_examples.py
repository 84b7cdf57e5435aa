"""The example scripts run end to end on CPU with tiny settings."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV = dict(os.environ, CUDA_VISIBLE_DEVICES="")


def _run(args, timeout=300):
    res = subprocess.run([sys.executable] + args, capture_output=True, text=True, timeout=timeout, env=ENV, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-1500:]
    return res.stdout


def test_mnist_example():
    out = _run(["examples/mnist.py", "--samples", "600", "--device", "cpu"])
    assert "epsilon" in out


def test_char_lstm_example():
    out = _run(["examples/char_lstm_classification.py", "--cell", "gru", "--epochs", "1", "--device", "cpu"])
    assert "accuracy" in out


def test_dcgan_example():
    out = _run(["examples/dcgan.py", "--steps", "2", "--device", "cpu"])
    assert "epsilon" in out


@pytest.mark.parametrize("script,extra", [("tensor_parallelism_toy.py", []), ("tensor_parallelism_llama.py", ["--sp", "--steps", "1"])])
def test_tensor_parallel_examples(script, extra):
    out = _run(["-m", "torch.distributed.run", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port",
                "29788", os.path.join("examples", script)] + extra, timeout=400)
    assert "step 0" in out


def test_cifar10_example():
    out = _run(["examples/cifar10.py", "--logical-batch", "64", "--physical-batch", "32", "--steps", "1", "--device", "cpu"])
    assert "epsilon" in out


def test_imdb_example():
    out = _run(["examples/imdb.py", "--epochs", "1", "--device", "cpu"])
    assert "epsilon spent" in out


def test_vision_benchmark_example():
    out = _run(["examples/vision_benchmark.py", "--device", "cpu", "--architecture", "cnn", "--batch-size", "16",
                "--steps", "2", "--modes", "none,hooks,ghost"])
    assert "of non-private" in out and "ghost" in out
