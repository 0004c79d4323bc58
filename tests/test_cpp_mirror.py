"""The C++ host mirror (include/rtensors_b200.hpp): compiles everywhere; on a GPU the restated
reference tests in tests/cpp/test_tensor_api.cpp must pass."""
import os
import subprocess

import pytest

import rtensors_b200 as rt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "rtensors_b200")


def _build(tmp_path, name="test_tensor_api"):
    rt.lib()  # the shared library must exist
    exe = str(tmp_path / name)
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-pthread", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", name + ".cpp"), "-o", exe,
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


def test_cpp_multi_gpu_case_compiles_and_links(tmp_path):
    _build(tmp_path, "test_mg_two_threads")


@pytest.mark.gpu
def test_cpp_two_ranks_in_one_process(tmp_path):
    """rtb_mg_* from compiled code, one host thread per device (prints "skipped" on a 1-GPU box)."""
    exe = _build(tmp_path, "test_mg_two_threads")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([exe], capture_output=True, text=True, timeout=180, env=env)
    assert p.returncode == 0, p.stdout + p.stderr
    assert "ok:" in p.stdout or "skipped" in p.stdout


def test_cpp_tape_compiles_and_links(tmp_path):
    _build(tmp_path, "test_grad_tape")


@pytest.mark.gpu
def test_cpp_tape_gradients_and_reference_models(tmp_path):
    """include/rtensors_b200_grad.hpp: analytic gradients in both modes, then the first four models of the
    reference's autograd test trained with SGD."""
    exe = _build(tmp_path, "test_grad_tape")
    p = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr
    assert "ok:" in p.stdout
