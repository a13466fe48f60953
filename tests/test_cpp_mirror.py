"""Builds and runs tests/cpp/test_mirror.cpp: the C++ host mirror of the reference's DmmvDispatch
(include/zinc_dmmv.hpp) over the C ABI. CPU run: layout helpers and the no-device error; GPU run: the
reference's error cases and one matvec."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "_build", "test_mirror")


def _build():
    from zinc_b200 import _lib

    _lib.lib()  # raises if the shared library has not been built
    os.makedirs(os.path.dirname(EXE), exist_ok=True)
    libdir = os.path.dirname(_lib.SO_PATH)
    cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "test_mirror.cpp"), "-o", EXE, "-L", libdir, "-lzinc_b200",
           "-Wl,-rpath," + libdir]
    subprocess.run(cmd, check=True, capture_output=True, text=True)


def _run():
    _build()
    r = subprocess.run([EXE], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout.strip()


def test_cpp_mirror_builds_and_reports_no_device():
    import torch

    out = _run()
    assert out == ("ok device" if torch.cuda.is_available() else "ok no-device")


@pytest.mark.gpu
def test_cpp_mirror_on_device():
    assert _run() == "ok device"
