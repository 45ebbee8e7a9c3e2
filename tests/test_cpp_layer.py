"""Runs the C++ operator-layer test program (tests/cpp/test_api.cpp): host-only checks here, the device
known-answer cases under the gpu marker."""
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
CPP = os.path.join(HERE, "cpp")
EXE = os.path.join(CPP, "test_api")


def _build():
    from phoenix_core_b200.csrc import build
    build.build()
    subprocess.check_call(["make", "-C", CPP, "test_api"], stdout=subprocess.DEVNULL)
    return EXE


def test_cpp_layer_host_side():
    exe = _build()
    res = subprocess.run([exe, "--cpu"], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr


@pytest.mark.gpu
def test_cpp_layer_on_device():
    exe = EXE if os.path.exists(EXE) else _build()
    res = subprocess.run([exe, "--gpu"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
