"""The C++ host mirror (include/rtensors_b200.hpp): compiles everywhere; on a GPU the restated
reference tests in tests/cpp/test_tensor_api.cpp must pass."""
import os
import subprocess

import pytest

import rtensors_b200 as rt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "rtensors_b200")


def _build(tmp_path):
    rt.lib()  # the shared library must exist
    exe = str(tmp_path / "test_tensor_api")
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "test_tensor_api.cpp"), "-o", exe,
           "-L", LIBDIR, "-lrt_b200", f"-Wl,-rpath,{LIBDIR}"]
    p = subprocess.run(cmd, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    return exe


def test_cpp_mirror_compiles_and_links(tmp_path):
    _build(tmp_path)


@pytest.mark.gpu
def test_cpp_mirror_reference_tests(tmp_path):
    exe = _build(tmp_path)
    p = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr
    assert "ok:" in p.stdout
