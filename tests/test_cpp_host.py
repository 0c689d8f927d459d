"""The C++ host layer (anode_b200/host/anode_ops.hpp): builds the test program of tests/cpp and,
on a GPU, runs it.  Without a GPU the program must still link, load both libraries and report that
it found no device."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "tests", "cpp")
BIN = os.path.join(CPP, "test_host_ops")


def build():
    import __graft_entry__
    __graft_entry__.build()          # library, oracle, then this program
    assert os.path.exists(BIN)


def test_cpp_host_layer_builds_and_loads():
    build()
    import torch
    if torch.cuda.is_available():
        pytest.skip("covered by the GPU test")
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=120)
    assert r.returncode == 2 and "no CUDA device" in r.stderr, (r.returncode, r.stdout, r.stderr)


@pytest.mark.gpu
def test_cpp_host_layer_on_gpu():
    build()
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 tests failed" in r.stdout
